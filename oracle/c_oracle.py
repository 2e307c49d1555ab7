"""ctypes front-end of the C oracle (``qlora_oracle.c``).

TEST INFRASTRUCTURE: a checker for the CUDA path, never the thing shipped.
All arrays are numpy; shapes follow the reference (row-major flat f32).
Each wrapper names the reference function it restates.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "_build", "liboracle.so")

DOUBLE_QUANT_BLOCK = 256  # qlora-core/src/quant.rs:50
NF4_ZERO_CODE = 7  # qlora-core/src/quant.rs:47


def build(force: bool = False) -> str:
    """Compile the oracle with the recipe in oracle/Makefile (gcc only)."""
    src = os.path.join(_HERE, "qlora_oracle.c")
    if force or not os.path.exists(_SO) or os.path.getmtime(_SO) < os.path.getmtime(src):
        subprocess.check_call(["make", "-s", "-C", _HERE], stdout=subprocess.DEVNULL)
    return _SO


_lib = None


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(_SO):
            build()
        _lib = C.CDLL(_SO)
        _declare(_lib)
    return _lib


_f32p = np.ctypeslib.ndpointer(dtype=np.float32, flags="C_CONTIGUOUS")
_u8p = np.ctypeslib.ndpointer(dtype=np.uint8, flags="C_CONTIGUOUS")
_sz = C.c_size_t


def _declare(l):
    l.orc_nf4_levels.restype = C.POINTER(C.c_float)
    l.orc_nearest_nf4_code.restype = C.c_uint8
    l.orc_nearest_nf4_code.argtypes = [C.c_float, C.c_float]
    l.orc_nf4_code_of_target.restype = C.c_uint8
    l.orc_nf4_code_of_target.argtypes = [C.c_float]
    l.orc_nf4_codes_of_target_bits.argtypes = [C.c_uint32, _sz, _u8p, C.c_int]
    l.orc_double_quantize_scales.argtypes = [_f32p, _sz, _u8p, _f32p]
    l.orc_quantize_nf4.argtypes = [_f32p, _sz, _sz, C.c_int, _u8p, _f32p, C.c_void_p, C.c_void_p]
    l.orc_block_scales_dq.argtypes = [_u8p, _f32p, _sz, _f32p]
    l.orc_dequantize.argtypes = [_u8p, _f32p, _sz, _sz, _f32p]
    for name in ("orc_matmul", "orc_matmul_trans_a", "orc_matmul_trans_b"):
        getattr(l, name).argtypes = [_f32p, _f32p, _sz, _sz, _sz, _f32p, C.c_int]
    l.orc_lora_scale.restype = C.c_float
    l.orc_lora_scale.argtypes = [C.c_float, _sz]
    l.orc_lora_forward.argtypes = [_f32p, _sz, _f32p, _f32p, _sz, _sz, _sz, C.c_float, _f32p, C.c_int]
    l.orc_qlora_forward.argtypes = [_f32p, _sz, _f32p, _sz, _sz, C.c_void_p, C.c_void_p, _sz, C.c_float, _f32p, C.c_int]
    l.orc_qlora_backward.argtypes = [_f32p, _f32p, _sz, _f32p, _sz, _sz, C.c_void_p, C.c_void_p, _sz, C.c_float,
                                     _f32p, C.c_void_p, C.c_void_p, C.c_int]
    l.orc_quantize_block_i8.restype = C.c_float
    l.orc_quantize_block_i8.argtypes = [_f32p, _sz, _u8p]
    l.orc_dequant_block_i8.argtypes = [_u8p, C.c_float, _f32p, _sz]
    l.orc_adam8bit_step_param.restype = _sz
    l.orc_adam8bit_step_param.argtypes = [C.c_float, C.c_float, C.c_float, C.c_float, _sz, _sz,
                                          C.POINTER(C.c_uint64), _sz, _u8p, _f32p, _u8p, _f32p, _f32p, _f32p]
    l.orc_adam_bias_corrections.argtypes = [C.c_float, C.c_float, C.c_uint64, C.POINTER(C.c_float), C.POINTER(C.c_float)]
    l.orc_max_threads.restype = C.c_int


def _f32(a):
    return np.ascontiguousarray(a, dtype=np.float32).reshape(-1)


def _ptr(a):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


def nf4_levels() -> np.ndarray:
    """qlora-core/src/quant.rs:27-44"""
    p = lib().orc_nf4_levels()
    return np.array([p[i] for i in range(16)], dtype=np.float32)


def max_threads() -> int:
    return int(lib().orc_max_threads())


class Quantized:
    """Result of `quantize_nf4`: mirrors QuantizedTensor's fields (quant.rs:93-101)."""

    def __init__(self, rows, cols, block_size, codes, scales_f32, absmax_codes, absmax2):
        self.rows, self.cols, self.block_size = rows, cols, block_size
        self.codes = codes
        self.scales_f32 = scales_f32  # first-level fp32 absmax (always kept for inspection)
        self.absmax_codes = absmax_codes  # None without double quant
        self.absmax2 = absmax2
        self.double_quant = absmax_codes is not None

    @property
    def num_blocks(self):
        return len(self.scales_f32)

    def block_scales(self) -> np.ndarray:
        """quant.rs:212-221"""
        if not self.double_quant:
            return self.scales_f32.copy()
        out = np.empty(self.num_blocks, np.float32)
        lib().orc_block_scales_dq(self.absmax_codes, self.absmax2, self.num_blocks, out)
        return out

    def dequantize(self) -> np.ndarray:
        """quant.rs:157-167"""
        return dequantize(self.codes, self.block_scales(), self.rows * self.cols, self.block_size)

    def storage_bytes(self) -> int:
        """quant.rs:229-235"""
        if self.double_quant:
            return len(self.codes) + len(self.absmax_codes) + 4 * len(self.absmax2)
        return len(self.codes) + 4 * len(self.scales_f32)


def quantize_nf4(w, rows, cols, block_size=64, double_quant=True) -> Quantized:
    """QuantizedTensor::quantize — quant.rs:104-154 (+ :283-299 for double quant)."""
    w = _f32(w)
    n = rows * cols
    if block_size == 0:
        raise ValueError("invalid config: block_size must be > 0")
    if w.size != n:
        raise ValueError(f"shape mismatch: weights.len() = {w.size} but rows*cols = {n}")
    nb = (n + block_size - 1) // block_size
    codes = np.zeros((n + 1) // 2, np.uint8)
    scales = np.zeros(nb, np.float32)
    ac = a2 = None
    if double_quant:
        ac = np.zeros(nb, np.uint8)
        a2 = np.zeros((nb + DOUBLE_QUANT_BLOCK - 1) // DOUBLE_QUANT_BLOCK, np.float32)
    lib().orc_quantize_nf4(w, n, block_size, int(bool(double_quant)), codes, scales, _ptr(ac), _ptr(a2))
    return Quantized(rows, cols, block_size, codes, scales, ac, a2)


def dequantize(codes, scales, n, block_size) -> np.ndarray:
    out = np.empty(n, np.float32)
    lib().orc_dequantize(np.ascontiguousarray(codes, np.uint8), _f32(scales), n, block_size, out)
    return out


def nearest_nf4_code(w: float, absmax: float) -> int:
    """quant.rs:263-278"""
    return int(lib().orc_nearest_nf4_code(np.float32(w), np.float32(absmax)))


def nf4_code_of_target(t: float) -> int:
    return int(lib().orc_nf4_code_of_target(np.float32(t)))


def nf4_codes_of_target_bits(first_bits: int, count: int, threads: int = 0) -> np.ndarray:
    """The 16-way scan (quant.rs:263-278) for `count` consecutive fp32 bit patterns read as targets,
    two codes per byte (low nibble first)."""
    out = np.empty((count + 1) // 2, np.uint8)
    lib().orc_nf4_codes_of_target_bits(first_bits, count, out, threads or max(max_threads(), len(os.sched_getaffinity(0))))
    return out


def block_scales_dq(absmax_codes, absmax2) -> np.ndarray:
    """quant.rs:212-221 on raw parts: (code as i8 as f32) / 127 * absmax2[block / 256]."""
    ac = np.ascontiguousarray(absmax_codes, np.uint8)
    out = np.empty(ac.size, np.float32)
    lib().orc_block_scales_dq(ac, _f32(absmax2), ac.size, out)
    return out


def matmul(a, b, m, k, n, threads=1):
    """lora.rs:129-142"""
    c = np.empty(m * n, np.float32)
    lib().orc_matmul(_f32(a), _f32(b), m, k, n, c, threads)
    return c


def matmul_trans_a(a, b, m, k, n, threads=1):
    """lora.rs:148-162 — C(k,n) = A(m,k)^T · B(m,n)"""
    c = np.empty(k * n, np.float32)
    lib().orc_matmul_trans_a(_f32(a), _f32(b), m, k, n, c, threads)
    return c


def matmul_trans_b(a, b, m, k, n, threads=1):
    """lora.rs:169-183 — C(m,n) = A(m,k) · B(n,k)^T"""
    c = np.empty(m * n, np.float32)
    lib().orc_matmul_trans_b(_f32(a), _f32(b), m, k, n, c, threads)
    return c


def lora_forward(x, batch, a, b, in_dim, out_dim, r, alpha, threads=1):
    """LoraAdapter::forward — lora.rs:86-103"""
    out = np.empty(batch * out_dim, np.float32)
    lib().orc_lora_forward(_f32(x), batch, _f32(a), _f32(b), in_dim, out_dim, r, alpha, out, threads)
    return out


def qlora_forward(x, batch, w_deq, out_dim, in_dim, a=None, b=None, r=0, alpha=0.0, threads=1):
    """QloraLinear::forward — qlora.rs:86-107 (w_deq = weight.dequantize())."""
    y = np.empty(batch * out_dim, np.float32)
    a_ = _f32(a) if r else None
    b_ = _f32(b) if r else None
    lib().orc_qlora_forward(_f32(x), batch, _f32(w_deq), out_dim, in_dim, _ptr(a_), _ptr(b_), r, alpha, y, threads)
    return y


def qlora_backward(x, dy, batch, w_deq, out_dim, in_dim, a=None, b=None, r=0, alpha=0.0, threads=1):
    """QloraLinear::backward — qlora.rs:116-165.  Returns (grad_x, grad_a|None, grad_b|None)."""
    gx = np.empty(batch * in_dim, np.float32)
    ga = np.empty(r * in_dim, np.float32) if r else None
    gb = np.empty(out_dim * r, np.float32) if r else None
    a_ = _f32(a) if r else None
    b_ = _f32(b) if r else None
    lib().orc_qlora_backward(_f32(x), _f32(dy), batch, _f32(w_deq), out_dim, in_dim, _ptr(a_), _ptr(b_), r, alpha,
                             gx, _ptr(ga), _ptr(gb), threads)
    return gx, ga, gb


def quantize_block_i8(x):
    """optim.rs:84-94"""
    x = _f32(x)
    codes = np.zeros(x.size, np.uint8)
    s = lib().orc_quantize_block_i8(x, x.size, codes)
    return codes, np.float32(s)


def dequant_block_i8(codes, absmax):
    """optim.rs:96-100"""
    codes = np.ascontiguousarray(codes, np.uint8)
    out = np.empty(codes.size, np.float32)
    lib().orc_dequant_block_i8(codes, np.float32(absmax), out, codes.size)
    return out


def adam_bias_corrections(beta1, beta2, step):
    b1, b2 = C.c_float(), C.c_float()
    lib().orc_adam_bias_corrections(np.float32(beta1), np.float32(beta2), step, C.byref(b1), C.byref(b2))
    return np.float32(b1.value), np.float32(b2.value)


class Adam8bit:
    """Adam8bit — optim.rs:143-204; per-tensor state as ParamState (optim.rs:104-132)."""

    def __init__(self, lr=1e-3, beta1=0.9, beta2=0.999, eps=1e-8, block_size=256, max_resident_pages=None):
        lr, beta1, beta2, eps = (np.float32(v) for v in (lr, beta1, beta2, eps))
        if not (lr > 0 and np.isfinite(lr)):
            raise ValueError("invalid config: lr must be positive and finite")
        if not (0.0 <= beta1 < 1.0) or not (0.0 <= beta2 < 1.0):
            raise ValueError("invalid config: betas must be in (0, 1)")
        if max_resident_pages is None:
            max_resident_pages = (1 << 64) - 1
        if block_size == 0 or max_resident_pages == 0:
            raise ValueError("invalid config: block_size and max_resident_pages must be > 0")
        self.cfg = (lr, beta1, beta2, eps, block_size, max_resident_pages)
        self.states = []

    def _new_state(self, numel):
        bs = self.cfg[4]
        nb = (numel + bs - 1) // bs
        return dict(numel=numel, m_codes=np.zeros(numel, np.uint8), v_codes=np.zeros(numel, np.uint8),
                    m_scales=np.zeros(nb, np.float32), v_scales=np.zeros(nb, np.float32), step=C.c_uint64(0))

    def step(self, params, grads):
        """params: list of float32 arrays updated in place. Returns (pages_streamed, state_bytes)."""
        if len(params) != len(grads):
            raise ValueError(f"shape mismatch: params.len() = {len(params)} but grads.len() = {len(grads)}")
        lr, b1, b2, eps, bs, pages = self.cfg
        streamed = 0
        for i, (p, g) in enumerate(zip(params, grads)):
            if p.size != np.asarray(g).size:
                raise ValueError(f"shape mismatch: param {i}: len = {p.size} but grad len = {np.asarray(g).size}")
            if len(self.states) <= i:
                self.states.append(self._new_state(p.size))
            if self.states[i]["numel"] != p.size:
                self.states[i] = self._new_state(p.size)
            st = self.states[i]
            assert p.dtype == np.float32 and p.flags["C_CONTIGUOUS"]
            streamed += lib().orc_adam8bit_step_param(lr, b1, b2, eps, bs, min(pages, (1 << 63) - 1), C.byref(st["step"]),
                                                       p.size, st["m_codes"], st["m_scales"], st["v_codes"],
                                                       st["v_scales"], p.reshape(-1), _f32(g))
        return streamed, self.state_bytes()

    def state_bytes(self):
        return sum(2 * s["numel"] + 8 * len(s["m_scales"]) for s in self.states)
