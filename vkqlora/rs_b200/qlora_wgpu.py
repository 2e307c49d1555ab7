"""Drop-in for the reference's PyO3 module `qlora_wgpu` (qlora-python/src/lib.rs:301-310).

Same functions, classes, signatures and error behaviour (every failure is a ValueError, as
qlora-python/src/lib.rs:20-22 maps every QloraError to PyValueError); all data are flat row-major
Python lists of floats, exactly as in the reference.  Everything executes on the GPU through
libqlora_cuda.so — `use_gpu` is accepted for compatibility and ignored (there is no CPU path).

Use as:  `from vkqlora.rs_b200 import qlora_wgpu`  or put this package directory's parent on
sys.path and `import qlora_wgpu` via the alias installed by `install_alias()`.
"""
from __future__ import annotations

import sys
from typing import List, Optional

import numpy as np

from . import Adam8bit, AdamConfig, LoraAdapter, QloraLinear, QuantConfig, QuantizedTensor

__all__ = ["quantize_nf4", "qlora_linear_forward", "qlora_linear_backward", "QuantizedWeight", "BackwardOut",
           "PagedAdam"]


class QuantizedWeight:
    """qlora-python/src/lib.rs:29-78.  `scales` are the decoded fp32 block scales (double
    quantisation is decoded on export, lib.rs:100-101).  The handle of the device-resident tensor
    (with its 8-bit absmax codes) is kept alongside so the kernels read the compact form."""

    def __init__(self, rows, cols, block_size, double_quant, codes: bytes, scales: List[float], tensor=None):
        self.rows, self.cols, self.block_size, self.double_quant = rows, cols, block_size, double_quant
        self._codes = bytes(codes)
        self.scales = scales
        self._tensor = tensor  # QuantizedTensor with the original scale store, or None

    def codes_bytes(self) -> bytes:
        return self._codes

    @property
    def codes_list(self) -> List[int]:
        return list(self._codes)

    def dequantize(self) -> List[float]:
        """lib.rs:58-70: NF4_LEVELS[code] * scales[idx / block_size] on the exported fields (codes and decoded
        fp32 scales), computed on the GPU: the fields are rebuilt into a device tensor exactly as the forward
        and backward entry points do (lib.rs:181-188) and dequantised there (one fp32 multiply per element,
        bit-identical to the reference's loop)."""
        if len(self._codes) != (self.rows * self.cols + 1) // 2:
            raise ValueError("QuantizedWeight codes length does not match rows*cols")
        t = QuantizedTensor.from_raw_parts(self.rows, self.cols, self.block_size, self._codes, self.scales)
        return t.dequantize().tolist()

    def __repr__(self) -> str:
        return (f"QuantizedWeight(rows={self.rows}, cols={self.cols}, block_size={self.block_size}, "
                f"double_quant={'true' if self.double_quant else 'false'})")


def quantize_nf4(weights, rows: int, cols: int, block_size: int = 64, double_quant: bool = True) -> QuantizedWeight:
    """lib.rs:81-103"""
    q = QuantizedTensor.quantize(np.asarray(weights, np.float32), rows, cols, QuantConfig(block_size, double_quant))
    return QuantizedWeight(q.rows(), q.cols(), q.block_size(), q.uses_double_quant(), q.codes().tobytes(),
                           q.block_scales().tolist(), q)


def _rebuild_layer(weight: QuantizedWeight, lora_a, lora_b, lora_alpha) -> QloraLinear:
    """lib.rs:136-204"""
    in_dim, out_dim = weight.cols, weight.rows
    if lora_a is None and lora_b is None:
        r = 0
    elif lora_a is not None and lora_b is not None:
        if len(lora_a) % max(in_dim, 1) != 0:
            raise ValueError("lora_a length must be a multiple of in_dim")
        r = len(lora_a) // max(in_dim, 1)
        if len(lora_b) != out_dim * r:
            raise ValueError("lora_b length must equal out_dim * rank")
    else:
        raise ValueError("lora_a and lora_b must be given together")
    if len(weight._codes) != (out_dim * in_dim + 1) // 2:
        raise ValueError("QuantizedWeight codes length does not match rows*cols")
    # The reference rebuilds from (codes, decoded fp32 scales) -> ScaleStore::F32 (lib.rs:181-188).
    tensor = QuantizedTensor.from_raw_parts(weight.rows, weight.cols, weight.block_size, weight._codes, weight.scales)
    adapter = None
    if r:
        adapter = LoraAdapter(lora_a, lora_b, in_dim, out_dim, r, float(r) if lora_alpha is None else lora_alpha)
    return QloraLinear.from_quantized(tensor, adapter)


def qlora_linear_forward(x, batch: int, weight: QuantizedWeight, lora_a=None, lora_b=None, lora_alpha=None,
                         use_gpu: bool = False) -> List[float]:
    """lib.rs:115-133"""
    layer = _rebuild_layer(weight, lora_a, lora_b, lora_alpha)
    return layer.forward(np.asarray(x, np.float32), batch).tolist()


class BackwardOut:
    """lib.rs:239-247"""

    def __init__(self, grad_a, grad_b, grad_x):
        self.grad_a, self.grad_b, self.grad_x = grad_a, grad_b, grad_x


def qlora_linear_backward(x, dy, batch: int, weight: QuantizedWeight, lora_a=None, lora_b=None, lora_alpha=None,
                          use_gpu: bool = False) -> BackwardOut:
    """lib.rs:211-236"""
    layer = _rebuild_layer(weight, lora_a, lora_b, lora_alpha)
    g = layer.backward(np.asarray(x, np.float32), np.asarray(dy, np.float32), batch)
    return BackwardOut(None if g.grad_a is None else g.grad_a.tolist(),
                       None if g.grad_b is None else g.grad_b.tolist(), g.grad_x.tolist())


class PagedAdam:
    """lib.rs:258-298"""

    def __init__(self, lr=1e-3, beta1=0.9, beta2=0.999, eps=1e-8, block_size=256, max_resident_pages=None):
        self._opt = Adam8bit(AdamConfig(lr, beta1, beta2, eps, block_size, max_resident_pages))

    def step(self, params, grads) -> List[List[float]]:
        owned = [np.array(p, dtype=np.float32) for p in params]
        self._opt.step(owned, [np.asarray(g, np.float32) for g in grads])
        return [p.tolist() for p in owned]

    def state_bytes(self) -> int:
        return self._opt.state_bytes()


def install_alias() -> None:
    """Registers this module as top-level `qlora_wgpu`, so code written against the reference's
    Python package (`import qlora_wgpu`) runs unchanged."""
    sys.modules.setdefault("qlora_wgpu", sys.modules[__name__])
