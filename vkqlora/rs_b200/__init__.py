"""vkqlora.rs_b200 — host-side mirror of the reference's QloraLinear hot-path API over the
B200 CUDA library (libqlora_cuda.so, C ABI in include/qlora_cuda.h).

Names, argument meaning and error behaviour follow the reference crates:

  qlora-core   QuantConfig, QuantizedTensor, LoraAdapter, QloraLinear, QloraGrads,
               AdamConfig, Adam8bit, AdamStats, QloraError          (qlora-core/src/lib.rs:37-47)
  qlora-wgpu   GpuContext, gpu_dequantize, gpu_matmul, gpu_matmul_trans_a, gpu_matmul_trans_b,
               gpu_qlora_forward, gpu_qlora_backward                (qlora-wgpu/src/lib.rs:28-32)

Differences that are deliberate:
  * every operation runs on the GPU; there is no CPU path.  Where the reference accepts
    `ctx = None` and silently computes on the CPU (qlora-wgpu/src/kernels.rs:48-50), this
    package raises GpuError.
  * host data are numpy float32 arrays (flat, row-major) instead of Vec<f32>.
  * `*_dev` methods additionally accept raw device pointers (ints) for callers that keep
    activations in device memory (e.g. torch tensors: pass `t.data_ptr()`).

The Python module with the reference's PyO3 entry points is `vkqlora.rs_b200.qlora_wgpu`.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass
from typing import List, Optional, Sequence

import numpy as np

from . import _lib
from ._lib import (DTYPE_BF16, DTYPE_F32, PRECISION_AUTO, PRECISION_BF16, PRECISION_FP32_EXACT, PRECISION_TF32, GpuError,
                   InvalidConfig, QloraError, ShapeMismatch, check, lib)

__all__ = [
    "QloraError", "ShapeMismatch", "InvalidConfig", "GpuError", "QuantConfig", "QuantizedTensor", "LoraAdapter",
    "QloraLinear", "QloraGrads", "AdamConfig", "AdamStats", "Adam8bit", "GpuContext", "gpu_dequantize",
    "gpu_matmul", "gpu_matmul_trans_a", "gpu_matmul_trans_b", "gpu_qlora_forward", "gpu_qlora_backward",
    "NF4_LEVELS", "NF4_ZERO_CODE", "DOUBLE_QUANT_BLOCK", "DTYPE_F32", "DTYPE_BF16", "PRECISION_AUTO",
    "PRECISION_FP32_EXACT", "PRECISION_BF16", "PRECISION_TF32",
]

# qlora-core/src/quant.rs:27-50
NF4_LEVELS = np.array(
    [-1.0, -0.6961928009986877, -0.5250730514526367, -0.39491748809814453, -0.28444138169288635,
     -0.18477343022823334, -0.09105003625154495, 0.0, 0.07958029955625534, 0.16093020141124725,
     0.24611230194568634, 0.33791524171829224, 0.44070982933044434, 0.5626170039176941,
     0.7229568362236023, 1.0], dtype=np.float64).astype(np.float32)
NF4_ZERO_CODE = 7
DOUBLE_QUANT_BLOCK = 256


def _f32(a, name="array") -> np.ndarray:
    arr = np.ascontiguousarray(a, dtype=np.float32).reshape(-1)
    return arr


def _p(a: Optional[np.ndarray]):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


class GpuContext:
    """One CUDA device + stream (replaces qlora_wgpu::GpuContext, qlora-wgpu/src/context.rs:18-28)."""

    def __init__(self, device: int = 0):
        h = C.c_void_p()
        check(lib.qlc_ctx_create(device, C.byref(h)))
        self._h = h
        self.device = device

    @classmethod
    def try_new_blocking(cls, device: int = 0) -> "GpuContext":
        """GpuContext::try_new_blocking (context.rs:33).  The reference returns Ok(None) without an
        adapter so callers can fall back to the CPU; here that case raises GpuError."""
        return cls(device)

    def set_precision(self, precision: int) -> None:
        check(lib.qlc_ctx_set_precision(self._h, precision))

    def set_reserved_sms(self, sms: int) -> None:
        """SMs the one-wave weight GEMMs leave free for kernels of other streams (a collective that overlaps them)."""
        check(lib.qlc_ctx_set_reserved_sms(self._h, int(sms)))

    def synchronize(self) -> None:
        check(lib.qlc_ctx_synchronize(self._h))

    def profile_enable(self, on: bool) -> None:
        check(lib.qlc_ctx_profile_enable(self._h, int(on)))

    def profile_read(self, slot: int):
        """(total milliseconds, launches) of kernel slot `slot` since the last read."""
        ms, n = C.c_double(), C.c_uint64()
        check(lib.qlc_ctx_profile_read(self._h, slot, C.byref(ms), C.byref(n)))
        return ms.value, n.value

    def wait(self, ticket: int) -> None:
        """Blocks until the asynchronous host-buffer submission `ticket` has delivered its outputs."""
        check(lib.qlc_ctx_wait(self._h, ticket))

    def copy_to_host(self, dst: int, d_src: int, nbytes: int) -> None:
        """Device -> host copy in the context's stream order (complete after synchronize())."""
        check(lib.qlc_ctx_copy_to_host(self._h, dst, d_src, nbytes))

    def copy_to_device(self, d_dst: int, src: int, nbytes: int) -> None:
        check(lib.qlc_ctx_copy_to_device(self._h, d_dst, src, nbytes))

    @property
    def stream(self) -> int:
        return int(lib.qlc_ctx_stream(self._h) or 0)

    @property
    def launch_count(self) -> int:
        return int(lib.qlc_ctx_launch_count(self._h))

    def close(self) -> None:
        if getattr(self, "_h", None):
            lib.qlc_ctx_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


_default_ctx: Optional[GpuContext] = None


def default_context() -> GpuContext:
    """A process-wide context on device 0, created on first use."""
    global _default_ctx
    if _default_ctx is None:
        _default_ctx = GpuContext(0)
    return _default_ctx


def _require_ctx(ctx: Optional[GpuContext]) -> GpuContext:
    if ctx is None:
        raise GpuError(_lib.ERR_GPU, "gpu error: a GPU context is required (this backend has no CPU fallback)")
    return ctx


@dataclass(frozen=True)
class QuantConfig:
    """qlora-core/src/quant.rs:54-80"""
    block_size: int = 64
    double_quant: bool = True

    def validate(self) -> None:
        if self.block_size == 0:
            raise InvalidConfig(_lib.ERR_INVALID_CONFIG, "invalid config: block_size must be > 0")


class QuantizedTensor:
    """A row-major (rows, cols) weight quantised to NF4; payload lives in device memory
    (qlora-core/src/quant.rs:93-101)."""

    def __init__(self, handle, ctx: GpuContext):
        self._h = handle
        self._ctx = ctx
        info = _lib.QTensorInfo()
        check(lib.qlc_qtensor_get_info(self._h, C.byref(info)))
        self._info = info

    @classmethod
    def quantize(cls, weights, rows: int, cols: int, config: QuantConfig = QuantConfig(),
                 ctx: Optional[GpuContext] = None) -> "QuantizedTensor":
        """QuantizedTensor::quantize (quant.rs:104-154)."""
        ctx = ctx or default_context()
        w = _f32(weights)
        h = C.c_void_p()
        check(lib.qlc_quantize_nf4(ctx._h, _p(w), w.size, rows, cols, config.block_size, int(config.double_quant),
                                   C.byref(h)))
        return cls(h, ctx)

    @classmethod
    def quantize_dev(cls, d_weights: int, rows: int, cols: int, config: QuantConfig = QuantConfig(),
                     ctx: Optional[GpuContext] = None) -> "QuantizedTensor":
        """Same, reading rows*cols fp32 values from device memory (asynchronous)."""
        ctx = ctx or default_context()
        h = C.c_void_p()
        check(lib.qlc_quantize_nf4_dev(ctx._h, d_weights, rows, cols, config.block_size, int(config.double_quant),
                                       C.byref(h)))
        return cls(h, ctx)

    def requantize_dev(self, d_weights: int) -> None:
        """Quantise new fp32 device weights of the same shape into this tensor (no allocation, asynchronous)."""
        check(lib.qlc_qtensor_requantize_dev(self._ctx._h, self._h, d_weights))

    @classmethod
    def from_raw_parts(cls, rows: int, cols: int, block_size: int, codes, scales,
                       ctx: Optional[GpuContext] = None) -> "QuantizedTensor":
        """QuantizedTensor::from_raw_parts (quant.rs:171-207)."""
        ctx = ctx or default_context()
        c = np.ascontiguousarray(np.frombuffer(bytes(codes), dtype=np.uint8) if isinstance(codes, (bytes, bytearray))
                                 else np.asarray(codes, dtype=np.uint8))
        s = _f32(scales)
        h = C.c_void_p()
        check(lib.qlc_qtensor_from_raw_parts(ctx._h, rows, cols, block_size, _p(c), c.size, _p(s), s.size, C.byref(h)))
        return cls(h, ctx)

    @classmethod
    def from_double_quant_parts(cls, rows: int, cols: int, block_size: int, codes, absmax_codes, absmax2,
                                ctx: Optional[GpuContext] = None) -> "QuantizedTensor":
        """A double-quantised tensor from its stored payload (what codes() / absmax_codes() / absmax2() return):
        the 8-bit scales come back as they were, unlike from_raw_parts, which takes decoded fp32 scales."""
        ctx = ctx or default_context()
        c = np.ascontiguousarray(np.frombuffer(bytes(codes), dtype=np.uint8) if isinstance(codes, (bytes, bytearray))
                                 else np.asarray(codes, dtype=np.uint8))
        ac = np.ascontiguousarray(absmax_codes, dtype=np.uint8).reshape(-1)
        a2 = _f32(absmax2)
        h = C.c_void_p()
        check(lib.qlc_qtensor_from_double_quant_parts(ctx._h, rows, cols, block_size, _p(c), c.size, _p(ac), ac.size,
                                                      _p(a2), a2.size, C.byref(h)))
        return cls(h, ctx)

    # accessors, quant.rs:224-258
    def rows(self) -> int: return self._info.rows
    def cols(self) -> int: return self._info.cols
    def block_size(self) -> int: return self._info.block_size
    def num_elements(self) -> int: return self._info.num_elements
    def num_blocks(self) -> int: return self._info.num_blocks
    def storage_bytes(self) -> int: return self._info.storage_bytes
    def uses_double_quant(self) -> bool: return bool(self._info.double_quant)

    def codes(self) -> np.ndarray:
        out = np.empty(self._info.codes_len, np.uint8)
        check(lib.qlc_qtensor_codes(self._h, _p(out), out.size))
        return out

    def absmax_codes(self) -> np.ndarray:
        out = np.empty(self._info.num_blocks, np.uint8)
        check(lib.qlc_qtensor_absmax_codes(self._h, _p(out), out.size))
        return out

    def absmax2(self) -> np.ndarray:
        out = np.empty(self._info.absmax2_len, np.float32)
        check(lib.qlc_qtensor_absmax2(self._h, _p(out), out.size))
        return out

    def block_scales(self) -> np.ndarray:
        """quant.rs:212-221"""
        out = np.empty(self._info.num_blocks, np.float32)
        check(lib.qlc_qtensor_block_scales(self._h, _p(out), out.size))
        return out

    def dequantize(self) -> np.ndarray:
        """quant.rs:157-167 (bit-exact)."""
        out = np.empty(self._info.num_elements, np.float32)
        check(lib.qlc_dequantize(self._ctx._h, self._h, _p(out), out.size))
        return out

    def dequantize_dev(self, d_out: int, dtype: int = DTYPE_F32) -> None:
        check(lib.qlc_dequantize_dev(self._ctx._h, self._h, d_out, dtype))

    def device_ptrs(self):
        ptrs = [C.c_void_p() for _ in range(4)]
        check(lib.qlc_qtensor_device_ptrs(self._h, *[C.byref(p) for p in ptrs]))
        return tuple(p.value for p in ptrs)

    def close(self) -> None:
        if getattr(self, "_h", None):
            lib.qlc_qtensor_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class LoraAdapter:
    """A:(r, in_dim), B:(out_dim, r), scaling alpha/r (qlora-core/src/lora.rs:17-123)."""

    def __init__(self, a, b, in_dim: int, out_dim: int, r: int, alpha: float):
        a, b = _f32(a), _f32(b)
        if r == 0:
            raise InvalidConfig(_lib.ERR_INVALID_CONFIG, "invalid config: rank r must be > 0")
        if a.size != r * in_dim:
            raise ShapeMismatch(_lib.ERR_SHAPE_MISMATCH, f"shape mismatch: a.len() = {a.size} but r*in_dim = {r * in_dim}")
        if b.size != out_dim * r:
            raise ShapeMismatch(_lib.ERR_SHAPE_MISMATCH, f"shape mismatch: b.len() = {b.size} but out_dim*r = {out_dim * r}")
        self._in, self._out, self._r, self._alpha = in_dim, out_dim, r, float(alpha)
        self._a, self._b = a.copy(), b.copy()
        self._layer: Optional["QloraLinear"] = None

    def scale(self) -> float:
        return float(np.float32(self._alpha) / np.float32(self._r))

    def set_weights(self, a, b) -> None:
        """lora.rs:70-83"""
        a, b = _f32(a), _f32(b)
        if a.size != self._a.size or b.size != self._b.size:
            raise ShapeMismatch(_lib.ERR_SHAPE_MISMATCH,
                                f"shape mismatch: set_weights: got ({a.size}, {b.size}), expected ({self._a.size}, {self._b.size})")
        self._a[:] = a
        self._b[:] = b
        if self._layer is not None:
            check(lib.qlc_layer_set_weights(self._layer._h, _p(self._a), a.size, _p(self._b), b.size))

    def in_dim(self) -> int: return self._in
    def out_dim(self) -> int: return self._out
    def rank(self) -> int: return self._r
    def alpha(self) -> float: return self._alpha
    def a(self) -> np.ndarray: return self._a
    def b(self) -> np.ndarray: return self._b


@dataclass
class QloraGrads:
    """qlora-core/src/qlora.rs:13-20"""
    grad_a: Optional[np.ndarray]
    grad_b: Optional[np.ndarray]
    grad_x: np.ndarray


class QloraLinear:
    """Frozen NF4 base weight + optional LoRA adapter (qlora-core/src/qlora.rs:33-183)."""

    def __init__(self, weight: QuantizedTensor, adapter: Optional[LoraAdapter], ctx: GpuContext):
        if adapter is not None and (adapter.in_dim() != weight.cols() or adapter.out_dim() != weight.rows()):
            # qlora.rs:71-80 (and :49-62 for `new`)
            raise ShapeMismatch(_lib.ERR_SHAPE_MISMATCH,
                                f"shape mismatch: adapter ({adapter.out_dim()}, {adapter.in_dim()}) vs weight "
                                f"({weight.rows()}, {weight.cols()})")
        self._ctx, self._weight, self._adapter = ctx, weight, adapter
        h = C.c_void_p()
        if adapter is None:
            check(lib.qlc_layer_create(ctx._h, weight._h, None, 0, None, 0, 0, 0.0, C.byref(h)))
        else:
            check(lib.qlc_layer_create(ctx._h, weight._h, _p(adapter._a), adapter._a.size, _p(adapter._b),
                                       adapter._b.size, adapter.rank(), adapter.alpha(), C.byref(h)))
            adapter._layer = self
        self._h = h

    @classmethod
    def new(cls, weight_fp32, out_dim: int, in_dim: int, quant: QuantConfig = QuantConfig(),
            adapter: Optional[LoraAdapter] = None, ctx: Optional[GpuContext] = None) -> "QloraLinear":
        """QloraLinear::new (qlora.rs:41-64): quantises immediately."""
        ctx = ctx or default_context()
        quant.validate()
        weight = QuantizedTensor.quantize(weight_fp32, out_dim, in_dim, quant, ctx)
        return cls(weight, adapter, ctx)

    @classmethod
    def from_quantized(cls, weight: QuantizedTensor, adapter: Optional[LoraAdapter] = None,
                       ctx: Optional[GpuContext] = None) -> "QloraLinear":
        """QloraLinear::from_quantized (qlora.rs:67-83)."""
        return cls(weight, adapter, ctx or weight._ctx)

    def forward(self, x, batch: int) -> np.ndarray:
        """QloraLinear::forward (qlora.rs:86-107) on host fp32 data."""
        x = _f32(x)
        y = np.empty(batch * self.out_dim(), np.float32)
        check(lib.qlc_qlora_forward(self._ctx._h, self._h, _p(x), x.size, batch, _p(y)))
        return y

    def backward(self, x, dy, batch: int) -> QloraGrads:
        """QloraLinear::backward (qlora.rs:116-165) on host fp32 data."""
        x, dy = _f32(x), _f32(dy)
        r = self._adapter.rank() if self._adapter else 0
        gx = np.empty(batch * self.in_dim(), np.float32)
        ga = np.empty(r * self.in_dim(), np.float32) if r else None
        gb = np.empty(self.out_dim() * r, np.float32) if r else None
        check(lib.qlc_qlora_backward(self._ctx._h, self._h, _p(x), x.size, _p(dy), dy.size, batch, _p(gx), _p(ga), _p(gb)))
        return QloraGrads(ga, gb, gx)

    def forward_host(self, x: np.ndarray, batch: int, dtype: int) -> np.ndarray:
        """Host buffers in `dtype` (bf16 as uint16 bit patterns); copies are part of the call."""
        es = np.uint16 if dtype == DTYPE_BF16 else np.float32
        x = np.ascontiguousarray(x, dtype=es).reshape(-1)
        if x.size != batch * self.in_dim():  # the C call takes no lengths: a short array would be read past its end
            raise ShapeMismatch(_lib.ERR_SHAPE_MISMATCH,
                                f"shape mismatch: x.len() = {x.size} but batch*in_dim = {batch * self.in_dim()}")
        y = np.empty(batch * self.out_dim(), es)
        check(lib.qlc_qlora_forward_host(self._ctx._h, self._h, _p(x), dtype, batch, _p(y)))
        return y

    def forward_backward_host(self, x: np.ndarray, dy: np.ndarray, batch: int, dtype: int):
        """Forward and backward of one batch in one call (X crosses the host link once): returns (y, QloraGrads).
        Host buffers in `dtype` (bf16 as uint16 bit patterns); copies are part of the call."""
        es = np.uint16 if dtype == DTYPE_BF16 else np.float32
        x = np.ascontiguousarray(x, dtype=es).reshape(-1)
        dy = np.ascontiguousarray(dy, dtype=es).reshape(-1)
        if x.size != batch * self.in_dim() or dy.size != batch * self.out_dim():
            raise ShapeMismatch(_lib.ERR_SHAPE_MISMATCH, "shape mismatch: x must hold batch*in_dim and dy batch*out_dim values")
        r = self._adapter.rank() if self._adapter else 0
        y, gx = np.empty(batch * self.out_dim(), es), np.empty(batch * self.in_dim(), es)
        ga = np.empty(r * self.in_dim(), np.float32) if r else None
        gb = np.empty(self.out_dim() * r, np.float32) if r else None
        check(lib.qlc_qlora_forward_backward_host(self._ctx._h, self._h, _p(x), _p(dy), dtype, batch, _p(y), _p(gx), _p(ga),
                                                  _p(gb)))
        return y, QloraGrads(ga, gb, gx)

    def forward_backward_host_async(self, x: int, dy: int, batch: int, dtype: int, y: int, grad_x: int,
                                    grad_a: Optional[int], grad_b: Optional[int]) -> int:
        """Queues forward + backward on HOST buffers given as addresses (pinned memory for real overlap) and returns
        a ticket for GpuContext.wait(); the buffers must stay valid and untouched until then."""
        t = C.c_uint64()
        check(lib.qlc_qlora_forward_backward_host_async(self._ctx._h, self._h, x, dy, dtype, batch, y, grad_x, grad_a, grad_b,
                                                        C.byref(t)))
        return int(t.value)

    def forward_dev(self, d_x: int, batch: int, d_y: int, dtype: int = DTYPE_BF16) -> None:
        check(lib.qlc_qlora_forward_dev(self._ctx._h, self._h, d_x, dtype, batch, d_y))

    def forward_dev_noalloc(self, d_x: int, batch: int, d_y: int) -> None:
        """bf16 forward that performs no device allocation (at most 8192 rows per call; its scratch is a
        fixed array inside the library shared by all calls on the device — do not overlap two of them)."""
        check(lib.qlc_qlora_forward_dev_noalloc(self._ctx._h, self._h, d_x, batch, d_y))

    def backward_dev(self, d_x: int, d_dy: int, batch: int, d_grad_x: int, d_grad_a: Optional[int],
                     d_grad_b: Optional[int], dtype: int = DTYPE_BF16) -> None:
        check(lib.qlc_qlora_backward_dev(self._ctx._h, self._h, d_x, d_dy, dtype, batch, d_grad_x, d_grad_a, d_grad_b))

    def adapter_dev(self):
        """(device pointer of fp32 A, device pointer of fp32 B): update in place, then adapter_updated()."""
        a, b = C.c_void_p(), C.c_void_p()
        check(lib.qlc_layer_adapter_dev(self._h, C.byref(a), C.byref(b)))
        return a.value, b.value

    def adapter_updated(self) -> None:
        check(lib.qlc_layer_adapter_updated(self._h))

    def train_step_dev(self, adam: "Adam8bit", d_x: int, d_dy: int, batch: int, d_grad_x: int,
                       dtype: int = DTYPE_BF16, comm: Optional["Comm"] = None) -> None:
        """backward -> (all-reduce) -> 8-bit Adam on A, B in place -> operand refresh, all on the device
        (what qlora-core/examples/train_lora.rs:41-46 does through host vectors)."""
        check(lib.qlc_train_step_dev(self._ctx._h, self._h, adam._h, comm._h if comm else None, d_x, d_dy, dtype, batch,
                                     d_grad_x))

    def grad_bucket(self):
        """(device pointer, float count) of the layer's contiguous grad_a‖grad_b bucket."""
        p, n = C.c_void_p(), C.c_size_t()
        check(lib.qlc_layer_grad_bucket(self._h, C.byref(p), C.byref(n)))
        return p.value, n.value

    def weight(self) -> QuantizedTensor: return self._weight
    def adapter(self) -> Optional[LoraAdapter]: return self._adapter
    def adapter_mut(self) -> Optional[LoraAdapter]: return self._adapter
    def in_dim(self) -> int: return self._weight.cols()
    def out_dim(self) -> int: return self._weight.rows()

    def close(self) -> None:
        if getattr(self, "_h", None):
            lib.qlc_layer_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


# ---- qlora-wgpu style free functions (qlora-wgpu/src/kernels.rs) ---------------------------------

def gpu_dequantize(ctx: Optional[GpuContext], q: QuantizedTensor) -> np.ndarray:
    """kernels.rs:44-103"""
    _require_ctx(ctx)
    out = np.empty(q.num_elements(), np.float32)
    check(lib.qlc_dequantize(ctx._h, q._h, _p(out), out.size))
    return out


def _gemm(fn, ctx, a, b, m, k, n, out_len):
    _require_ctx(ctx)
    a, b = _f32(a), _f32(b)
    c = np.empty(out_len, np.float32)
    check(fn(ctx._h, _p(a), a.size, _p(b), b.size, m, k, n, _p(c)))
    return c


def gpu_matmul(ctx, a, b, m: int, k: int, n: int) -> np.ndarray:
    """kernels.rs:140-176 — C(m,n) = A(m,k)·B(k,n)"""
    return _gemm(lib.qlc_matmul, ctx, a, b, m, k, n, m * n)


def gpu_matmul_trans_b(ctx, a, b, m: int, k: int, n: int) -> np.ndarray:
    """kernels.rs:180-216 — C(m,n) = A(m,k)·B(n,k)^T"""
    return _gemm(lib.qlc_matmul_trans_b, ctx, a, b, m, k, n, m * n)


def gpu_matmul_trans_a(ctx, a, b, m: int, k: int, n: int) -> np.ndarray:
    """kernels.rs:220-257 — C(k,n) = A(m,k)^T·B(m,n)"""
    return _gemm(lib.qlc_matmul_trans_a, ctx, a, b, m, k, n, k * n)


def gpu_qlora_forward(ctx: Optional[GpuContext], layer: QloraLinear, x, batch: int) -> np.ndarray:
    """kernels.rs:262-296"""
    _require_ctx(ctx)
    return layer.forward(x, batch)


def gpu_qlora_backward(ctx: Optional[GpuContext], layer: QloraLinear, x, dy, batch: int) -> QloraGrads:
    """kernels.rs:301-353"""
    _require_ctx(ctx)
    return layer.backward(x, dy, batch)


# ---- paged 8-bit Adam (qlora-core/src/optim.rs) -----------------------------------------------------

@dataclass
class AdamConfig:
    """optim.rs:33-58; max_resident_pages=None means usize::MAX (fully resident)."""
    lr: float = 1e-3
    beta1: float = 0.9
    beta2: float = 0.999
    eps: float = 1e-8
    block_size: int = 256
    max_resident_pages: Optional[int] = None


@dataclass
class AdamStats:
    """optim.rs:136-141"""
    pages_streamed: int
    state_bytes: int


COMM_ID_BYTES = 128


class Comm:
    """NCCL communicator bound to a context (one process per GPU).  The reference has no multi-device
    path; this is the exchange step of the token-sharded run: the sum of the LoRA gradients over ranks.

    Rank 0 calls Comm.unique_id() and hands the bytes to the other ranks over any host channel; every
    rank then constructs Comm(ctx, nranks, rank, id) (collective)."""

    def __init__(self, ctx: GpuContext, nranks: int, rank: int, unique_id: bytes):
        if len(unique_id) != COMM_ID_BYTES:
            raise InvalidConfig(2, f"invalid config: the communicator id has {COMM_ID_BYTES} bytes, got {len(unique_id)}")
        self._ctx = ctx
        buf = (C.c_ubyte * COMM_ID_BYTES).from_buffer_copy(unique_id)
        h = C.c_void_p()
        check(lib.qlc_comm_init(ctx._h, nranks, rank, buf, COMM_ID_BYTES, C.byref(h)))
        self._h = h
        self.nranks, self.rank = nranks, rank

    @staticmethod
    def unique_id() -> bytes:
        buf = (C.c_ubyte * COMM_ID_BYTES)()
        check(lib.qlc_comm_unique_id(buf, COMM_ID_BYTES))
        return bytes(buf)

    def allreduce_sum_f32(self, d_buf: int, count: int) -> None:
        """In-place sum over ranks of `count` floats at device pointer d_buf, in stream order."""
        check(lib.qlc_comm_allreduce_sum_f32(self._h, d_buf, count))

    def allreduce_lora_grads(self, layer: "QloraLinear") -> None:
        check(lib.qlc_allreduce_lora_grads(self._h, layer._h))

    def close(self) -> None:
        if getattr(self, "_h", None):
            lib.qlc_comm_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class Adam8bit:
    """optim.rs:143-204"""

    def __init__(self, config: AdamConfig = AdamConfig(), ctx: Optional[GpuContext] = None):
        self._ctx = ctx or default_context()
        self._block_size = config.block_size
        c = _lib.AdamConfig(config.lr, config.beta1, config.beta2, config.eps, config.block_size,
                            _lib.SIZE_MAX if config.max_resident_pages is None else config.max_resident_pages)
        h = C.c_void_p()
        check(lib.qlc_adam_create(self._ctx._h, C.byref(c), C.byref(h)))
        self._h = h

    def step(self, params: List[np.ndarray], grads: Sequence) -> AdamStats:
        """Adam8bit::step (optim.rs:164-199); `params` (float32 arrays) are updated in place."""
        if len(params) != len(grads):
            raise ShapeMismatch(_lib.ERR_SHAPE_MISMATCH,
                                f"shape mismatch: params.len() = {len(params)} but grads.len() = {len(grads)}")
        n = len(params)
        for p in params:
            if not (isinstance(p, np.ndarray) and p.dtype == np.float32 and p.flags["C_CONTIGUOUS"]):
                raise InvalidConfig(_lib.ERR_INVALID_CONFIG, "invalid config: params must be contiguous float32 arrays")
        gs = [_f32(g) for g in grads]
        pp = (C.c_void_p * n)(*[p.ctypes.data for p in params])
        gp = (C.c_void_p * n)(*[g.ctypes.data for g in gs])
        pl = (C.c_size_t * n)(*[p.size for p in params])
        gl = (C.c_size_t * n)(*[g.size for g in gs])
        st = _lib.AdamStats()
        check(lib.qlc_adam_step(self._h, n, pp, pl, gp, gl, C.byref(st)))
        return AdamStats(st.pages_streamed, st.state_bytes)

    def step_dev(self, d_params: Sequence[int], d_grads: Sequence[int], lens: Sequence[int]) -> AdamStats:
        n = len(d_params)
        pp = (C.c_void_p * n)(*d_params)
        gp = (C.c_void_p * n)(*d_grads)
        ll = (C.c_size_t * n)(*lens)
        st = _lib.AdamStats()
        check(lib.qlc_adam_step_dev(self._h, n, pp, gp, ll, C.byref(st)))
        return AdamStats(st.pages_streamed, st.state_bytes)

    def set_fast_math(self, on: bool) -> None:
        """Opt into hardware-approximate arithmetic (parameters ~1e-6 relative per step instead of bit-exact)."""
        check(lib.qlc_adam_set_fast_math(self._h, int(on)))

    def state_bytes(self) -> int:
        return int(lib.qlc_adam_state_bytes(self._h))

    def get_state(self, index: int):
        numel, step = C.c_size_t(), C.c_uint64()
        check(lib.qlc_adam_get_state(self._h, index, C.byref(numel), C.byref(step), None, None, None, None))
        n = numel.value
        mc, vc = np.empty(n, np.uint8), np.empty(n, np.uint8)
        nb = (n + self._block_size - 1) // self._block_size
        ms, vs = np.empty(nb, np.float32), np.empty(nb, np.float32)
        check(lib.qlc_adam_get_state(self._h, index, None, None, _p(mc), _p(vc), _p(ms), _p(vs)))
        return dict(numel=n, step=step.value, m_codes=mc, v_codes=vc, m_scales=ms, v_scales=vs)

    def set_state(self, index: int, state: dict) -> None:
        """Restores what get_state(index) returned (checkpoint restore); states are restored in order."""
        mc = np.ascontiguousarray(state["m_codes"], np.uint8)
        vc = np.ascontiguousarray(state["v_codes"], np.uint8)
        ms, vs = _f32(state["m_scales"]), _f32(state["v_scales"])
        n = int(state["numel"])
        nb = (n + self._block_size - 1) // self._block_size
        if mc.size != n or vc.size != n or ms.size != nb or vs.size != nb:
            raise ShapeMismatch(_lib.ERR_SHAPE_MISMATCH, "shape mismatch: state arrays do not match numel / block_size")
        check(lib.qlc_adam_set_state(self._h, index, n, int(state["step"]), _p(mc), _p(vc), _p(ms), _p(vs)))

    def paging_info(self):
        vals = [C.c_size_t() for _ in range(4)]
        check(lib.qlc_adam_paging_info(self._h, *[C.byref(v) for v in vals]))
        return dict(device_bytes=vals[0].value, host_bytes=vals[1].value, h2d_bytes_last_step=vals[2].value,
                    d2h_bytes_last_step=vals[3].value)

    def close(self) -> None:
        if getattr(self, "_h", None):
            lib.qlc_adam_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
