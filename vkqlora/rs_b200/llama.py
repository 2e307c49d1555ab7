"""Host mirror of the reference's `qlora_model::LlamaModel` (qlora-model/src/llama.rs) over the C ABI
(`qlc_llama_*`): Llama decoder whose seven projections per block are NF4 QloraLinear layers on the GPU."""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass
from typing import Dict, Optional, Sequence, Tuple

import numpy as np

from . import Adam8bit, GpuContext, QuantConfig, default_context
from ._lib import check, lib

KINDS = ("q", "k", "v", "o", "gate", "up", "down")  # ProjKind, llama.rs:44-54


class _Config(C.Structure):
    _fields_ = [("hidden", C.c_size_t), ("layers", C.c_size_t), ("heads", C.c_size_t), ("kv_heads", C.c_size_t),
                ("intermediate", C.c_size_t), ("vocab", C.c_size_t), ("rms_eps", C.c_float), ("rope_theta", C.c_float)]


@dataclass
class LlamaConfig:
    """llama.rs:13-43"""
    hidden: int = 576
    layers: int = 30
    heads: int = 9
    kv_heads: int = 3
    intermediate: int = 1536
    vocab: int = 49152
    rms_eps: float = 1e-5
    rope_theta: float = 10000.0

    @classmethod
    def smollm_135m(cls) -> "LlamaConfig":
        return cls()

    @property
    def head_dim(self) -> int:
        return self.hidden // self.heads

    @property
    def kv_dim(self) -> int:
        return self.kv_heads * self.head_dim

    def proj_dims(self, kind: str) -> Tuple[int, int]:
        h, i, kv = self.hidden, self.intermediate, self.kv_dim
        return {"q": (h, h), "k": (kv, h), "v": (kv, h), "o": (h, h), "gate": (i, h), "up": (i, h), "down": (h, i)}[kind]


def _f32(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.float32)


def _u32(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.uint32)


class LlamaModel:
    def __init__(self, cfg: LlamaConfig, embed, final_norm, ctx: Optional[GpuContext] = None):
        self.cfg = cfg
        self._ctx = ctx or default_context()
        c = _Config(cfg.hidden, cfg.layers, cfg.heads, cfg.kv_heads, cfg.intermediate, cfg.vocab, cfg.rms_eps, cfg.rope_theta)
        e, n = _f32(embed).reshape(-1), _f32(final_norm).reshape(-1)
        if e.size != cfg.vocab * cfg.hidden or n.size != cfg.hidden:
            raise ValueError("shape mismatch: embed must be (vocab, hidden) and final_norm (hidden)")
        h = C.c_void_p()
        check(lib.qlc_llama_create(self._ctx._h, C.byref(c), e.ctypes.data, n.ctypes.data, C.byref(h)))
        self._h = h

    def set_layer(self, li: int, attn_norm, mlp_norm, weights: Dict[str, np.ndarray], quant: QuantConfig = QuantConfig(),
                  quantize: Optional[Sequence[str]] = None) -> None:
        """weights[kind]: (out, in) fp32, all seven kinds (llama.rs:250-297).  quantize=None: every projection is
        NF4-quantised.  quantize=("q", "v"): only those kinds are; the others stay raw fp32 matrices, as in the
        reference, which quantises adapter targets only (llama.rs:228-249)."""
        mats = []
        for k in KINDS:
            o, i = self.cfg.proj_dims(k)
            w = _f32(weights[k]).reshape(-1)
            if w.size != o * i:
                raise ValueError(f"shape mismatch: {k} weight has {w.size} values, expected {o}*{i}")
            mats.append(w)
        ptrs = (C.c_void_p * 7)(*[m.ctypes.data for m in mats])
        an, mn = _f32(attn_norm), _f32(mlp_norm)
        if quantize is None:
            check(lib.qlc_llama_set_layer(self._h, li, an.ctypes.data, mn.ctypes.data, ptrs, quant.block_size,
                                          int(quant.double_quant)))
        else:
            flags = (C.c_int * 7)(*[int(k in quantize) for k in KINDS])
            check(lib.qlc_llama_set_layer_mixed(self._h, li, an.ctypes.data, mn.ctypes.data, ptrs, flags, quant.block_size,
                                                int(quant.double_quant)))

    def attach_adapter(self, li: int, kind: str, a, b, rank: int, alpha: float) -> None:
        a, b = _f32(a).reshape(-1), _f32(b).reshape(-1)
        o, i = self.cfg.proj_dims(kind)
        if a.size != rank * i or b.size != o * rank:
            raise ValueError("shape mismatch: adapter a must be (r, in) and b (out, r)")
        check(lib.qlc_llama_attach_adapter(self._h, li, KINDS.index(kind), a.ctypes.data, b.ctypes.data, rank, alpha))

    def forward(self, ids, n_seq: int, seq_len: int) -> np.ndarray:
        """LlamaModel::forward (llama.rs:310-326) -> (n_seq*seq_len, vocab) logits."""
        ids = _u32(ids).reshape(-1)
        out = np.empty((n_seq * seq_len, self.cfg.vocab), np.float32)
        check(lib.qlc_llama_forward(self._h, ids.ctypes.data, n_seq, seq_len, out.ctypes.data))
        return out

    def backward(self, ids, dlogits, n_seq: int, seq_len: int) -> None:
        """LlamaModel::backward (llama.rs:385-412); gradients are read with adapter_grads()."""
        ids, d = _u32(ids).reshape(-1), _f32(dlogits).reshape(-1)
        check(lib.qlc_llama_backward(self._h, ids.ctypes.data, d.ctypes.data, n_seq, seq_len))

    def loss_backward(self, ids, targets, n_seq: int, seq_len: int) -> float:
        ids, t = _u32(ids).reshape(-1), _u32(targets).reshape(-1)
        loss = C.c_float()
        check(lib.qlc_llama_loss_backward(self._h, ids.ctypes.data, t.ctypes.data, n_seq, seq_len, C.byref(loss)))
        return float(loss.value)

    def train_step(self, adam: Adam8bit, ids, targets, n_seq: int, seq_len: int, want_loss: bool = True,
                   comm=None) -> Optional[float]:
        """One training step on this rank's sequences.  With `comm` (a Comm on the model's context) the step is the
        data-parallel one: gradients of the mean loss over ALL ranks' tokens, summed over the ranks before the
        optimiser step; the returned loss is this rank's mean."""
        ids, t = _u32(ids).reshape(-1), _u32(targets).reshape(-1)
        loss = C.c_float()
        lp = C.byref(loss) if want_loss else None
        if comm is None:
            check(lib.qlc_llama_train_step(self._h, adam._h, ids.ctypes.data, t.ctypes.data, n_seq, seq_len, lp))
        else:
            check(lib.qlc_llama_train_step_dp(self._h, adam._h, comm._h, ids.ctypes.data, t.ctypes.data, n_seq, seq_len, lp))
        return float(loss.value) if want_loss else None

    def adapter_grads(self, li: int, kind: str, rank: int):
        o, i = self.cfg.proj_dims(kind)
        ga, gb = np.empty((rank, i), np.float32), np.empty((o, rank), np.float32)
        check(lib.qlc_llama_adapter_grads(self._h, li, KINDS.index(kind), ga.ctypes.data, gb.ctypes.data))
        return ga, gb

    def adapter_weights(self, li: int, kind: str, rank: int):
        o, i = self.cfg.proj_dims(kind)
        a, b = np.empty((rank, i), np.float32), np.empty((o, rank), np.float32)
        check(lib.qlc_llama_adapter_weights(self._h, li, KINDS.index(kind), a.ctypes.data, b.ctypes.data))
        return a, b

    def dequantized_weight(self, li: int, kind: str) -> np.ndarray:
        """The fp32 weights the projection actually multiplies by (NF4 round trip of what set_layer was given)."""
        layer = lib.qlc_llama_projection(self._h, li, KINDS.index(kind))
        q = lib.qlc_layer_weight(layer)
        o, i = self.cfg.proj_dims(kind)
        out = np.empty(o * i, np.float32)
        check(lib.qlc_dequantize(self._ctx._h, q, out.ctypes.data, out.size))
        return out.reshape(o, i)

    def close(self) -> None:
        if getattr(self, "_h", None):
            lib.qlc_llama_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
