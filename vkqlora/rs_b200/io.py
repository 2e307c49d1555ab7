"""On-disk formats around the hot path.

* `.safetensors` in: header parsing with the reference's validation rules
  (qlora-io/src/safetensors.rs:25-76: u64 LE header length, JSON header, raw little-endian data;
  offsets must lie inside the data and match numel * itemsize), and loading a weight matrix
  straight into an NF4 QuantizedTensor: the checkpoint's BF16 / F16 / F32 bytes are uploaded as
  they are and widened on the GPU, so no fp32 copy of the model is ever built on the host.
* `.npz` out: adapters as stored (uncompressed) `<f4` arrays, the form `tools/npz2pt.py:28-32` and
  `qlora-io/src/npz.rs:46-104` read and write.
"""
from __future__ import annotations

import json
import mmap
import os
import struct
from typing import Dict, Iterable, Mapping, Optional, Tuple

import numpy as np

from . import QuantConfig, QuantizedTensor, GpuContext, default_context
from ._lib import DTYPE_BF16, DTYPE_F16, DTYPE_F32, InvalidConfig, ShapeMismatch, check, lib
import ctypes as C

# dtype -> (itemsize, numpy dtype of the raw storage)  (safetensors.rs:82-99)
_DTYPES = {"F32": (4, "<f4"), "F16": (2, "<f2"), "BF16": (2, "<u2"), "I32": (4, "<i4"), "I64": (8, "<i8"),
           "U8": (1, "u1"), "BOOL": (1, "u1")}
_QUANT_CODES = {"F32": DTYPE_F32, "BF16": DTYPE_BF16, "F16": DTYPE_F16}


class SafetensorsFile:
    """Memory-mapped `.safetensors` file: `entries[name] = (dtype, shape, start, end)`."""

    def __init__(self, path: str):
        self.path = path
        self._f = open(path, "rb")
        size = os.fstat(self._f.fileno()).st_size
        if size < 8:
            raise InvalidConfig(2, "invalid config: file smaller than safetensors header")
        self._mm = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ)
        (hlen,) = struct.unpack("<Q", self._mm[:8])
        if hlen > size - 8:
            raise InvalidConfig(2, "invalid config: safetensors header length exceeds file")
        try:
            header = json.loads(self._mm[8:8 + hlen].decode("utf-8"))
        except (UnicodeDecodeError, json.JSONDecodeError) as e:
            raise InvalidConfig(2, f"invalid config: safetensors header is not valid UTF-8 JSON ({e})")
        self._data_off = 8 + hlen
        data_len = size - self._data_off
        self.entries: Dict[str, Tuple[str, Tuple[int, ...], int, int]] = {}
        for name, meta in header.items():
            if name == "__metadata__":
                continue
            dtype, shape = meta["dtype"], tuple(int(d) for d in meta["shape"])
            start, end = (int(o) for o in meta["data_offsets"])
            if end < start or end > data_len:
                raise InvalidConfig(2, f"invalid config: tensor {name!r}: offsets [{start}, {end}) outside data (len {data_len})")
            if dtype not in _DTYPES:
                raise InvalidConfig(2, f"invalid config: unsupported safetensors dtype {dtype!r}")
            numel = int(np.prod(shape, dtype=np.int64)) if shape else 1
            if end - start != numel * _DTYPES[dtype][0]:
                raise ShapeMismatch(1, f"shape mismatch: tensor {name!r}: byte range {end - start} != elements {numel} * "
                                       f"itemsize {_DTYPES[dtype][0]}")
            self.entries[name] = (dtype, shape, start, end)

    def names(self) -> Iterable[str]:
        return self.entries.keys()

    def raw(self, name: str) -> np.ndarray:
        """The tensor's stored values, zero-copy (bf16 as uint16 bit patterns)."""
        dtype, shape, start, end = self.entries[name]
        return np.frombuffer(self._mm, dtype=_DTYPES[dtype][1], count=(end - start) // _DTYPES[dtype][0],
                             offset=self._data_off + start).reshape(shape)

    def to_f32(self, name: str) -> np.ndarray:
        """Values widened to float32 on the host, as the reference's reader returns them (safetensors.rs:82-99)."""
        dtype = self.entries[name][0]
        raw = self.raw(name)
        if dtype == "BF16":
            return (raw.astype(np.uint32) << 16).view(np.float32)
        if dtype == "BOOL":
            return (raw != 0).astype(np.float32)
        return raw.astype(np.float32)

    def quantize(self, name: str, config: QuantConfig = QuantConfig(), ctx: Optional[GpuContext] = None) -> QuantizedTensor:
        """NF4-quantise the 2-D weight `name` on the GPU from its stored dtype (F32 / BF16 / F16)."""
        dtype, shape, _, _ = self.entries[name]
        if len(shape) != 2:
            raise ShapeMismatch(1, f"shape mismatch: tensor {name!r} has shape {shape}, expected a 2-D weight")
        if dtype not in _QUANT_CODES:
            raise InvalidConfig(2, f"invalid config: cannot quantise a {dtype} tensor")
        if config.block_size == 0:
            raise InvalidConfig(2, "invalid config: block_size must be > 0")
        ctx = ctx or default_context()
        raw = np.ascontiguousarray(self.raw(name))
        h = C.c_void_p()
        check(lib.qlc_quantize_nf4_typed(ctx._h, raw.ctypes.data, _QUANT_CODES[dtype], shape[0], shape[1], config.block_size,
                                         int(config.double_quant), C.byref(h)))
        return QuantizedTensor(h, ctx)

    def close(self) -> None:
        if getattr(self, "_mm", None) is not None:
            self._mm.close()
            self._f.close()
            self._mm = None

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()


def write_safetensors(path: str, tensors: Mapping[str, np.ndarray]) -> None:
    """Minimal writer (F32 / F16 arrays, or uint16 arrays holding BF16 bit patterns when the name maps to
    ("BF16", array)) - used to build test fixtures and to persist dequantised results."""
    header, blobs, off = {}, [], 0
    for name, t in tensors.items():
        dtype = None
        if isinstance(t, tuple):
            dtype, t = t
        t = np.ascontiguousarray(t)
        if dtype is None:
            dtype = {np.dtype("<f4"): "F32", np.dtype("<f2"): "F16"}.get(t.dtype)
            if dtype is None:
                raise InvalidConfig(2, f"invalid config: cannot store dtype {t.dtype} (give (\"BF16\", uint16 array) for bf16)")
        b = t.tobytes()
        header[name] = {"dtype": dtype, "shape": list(t.shape), "data_offsets": [off, off + len(b)]}
        blobs.append(b)
        off += len(b)
    hj = json.dumps(header, separators=(",", ":")).encode("utf-8")
    hj += b" " * ((8 - len(hj) % 8) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(hj)))
        f.write(hj)
        for b in blobs:
            f.write(b)


def save_adapters_npz(path: str, adapters: Mapping[str, np.ndarray]) -> None:
    """Stored (uncompressed) `.npz` of `<f4` arrays, readable by `np.load`, `qlora-io`'s `read_npz` and
    `tools/npz2pt.py`.  `adapters` maps names (e.g. "layers.0.q_proj.lora_A") to arrays."""
    np.savez(path, **{k: np.ascontiguousarray(v, dtype="<f4") for k, v in adapters.items()})


def load_adapters_npz(path: str) -> Dict[str, np.ndarray]:
    with np.load(path) as z:
        return {k: np.ascontiguousarray(z[k], dtype=np.float32) for k in z.files}


# ---- persisted NF4 payloads and optimiser state -------------------------------------------------------------
# The reference has no on-disk form for either (it re-quantises the checkpoint at every start and keeps the
# optimiser state in memory only).  Both are stored `.npz` files of plain arrays, so any numpy can read them.

def save_quantized_npz(path: str, tensors: Mapping[str, QuantizedTensor]) -> None:
    """NF4 payloads as they live on the device: per tensor `<name>.shape` = (rows, cols, block_size), `<name>.codes`
    (packed nibbles, quant.rs:132-136) and either `<name>.absmax_codes` + `<name>.absmax2` (double quantisation,
    quant.rs:283-299) or `<name>.scales` (fp32 block scales).  4.127 bit per weight at block 64."""
    out = {}
    for name, q in tensors.items():
        out[f"{name}.shape"] = np.asarray([q.rows(), q.cols(), q.block_size()], dtype="<i8")
        out[f"{name}.codes"] = q.codes()
        if q.uses_double_quant():
            out[f"{name}.absmax_codes"] = q.absmax_codes()
            out[f"{name}.absmax2"] = np.ascontiguousarray(q.absmax2(), dtype="<f4")
        else:
            out[f"{name}.scales"] = np.ascontiguousarray(q.block_scales(), dtype="<f4")
    np.savez(path, **out)


def load_quantized_npz(path: str, ctx: Optional[GpuContext] = None) -> Dict[str, QuantizedTensor]:
    """The inverse of save_quantized_npz: the tensors come back bit for bit (codes, 8-bit scales, second-level
    absmax), without a quantisation pass."""
    ctx = ctx or default_context()
    res: Dict[str, QuantizedTensor] = {}
    with np.load(path) as z:
        names = sorted({k[: -len(".shape")] for k in z.files if k.endswith(".shape")})
        for name in names:
            rows, cols, block = (int(v) for v in z[f"{name}.shape"])
            if f"{name}.absmax_codes" in z.files:
                res[name] = QuantizedTensor.from_double_quant_parts(rows, cols, block, z[f"{name}.codes"],
                                                                    z[f"{name}.absmax_codes"], z[f"{name}.absmax2"], ctx)
            elif f"{name}.scales" in z.files:
                res[name] = QuantizedTensor.from_raw_parts(rows, cols, block, z[f"{name}.codes"], z[f"{name}.scales"], ctx)
            else:
                raise InvalidConfig(2, f"invalid config: {name} has neither absmax_codes nor scales in {path}")
    return res


def save_adam_state_npz(path: str, opt, n_tensors: int) -> None:
    """The 8-bit state of the first `n_tensors` parameter tensors of an Adam8bit (ParamState, optim.rs:104-112:
    m / v codes, their block scales, the step count), resident or paged."""
    out = {"n_tensors": np.asarray([n_tensors], dtype="<i8")}
    for i in range(n_tensors):
        st = opt.get_state(i)
        out[f"{i}.meta"] = np.asarray([st["numel"], st["step"]], dtype="<i8")
        for k in ("m_codes", "v_codes"):
            out[f"{i}.{k}"] = st[k]
        for k in ("m_scales", "v_scales"):
            out[f"{i}.{k}"] = np.ascontiguousarray(st[k], dtype="<f4")
    np.savez(path, **out)


def load_adam_state_npz(path: str, opt) -> int:
    """Restores save_adam_state_npz's states into `opt` in order (an optimiser built with the same block size);
    the next step continues the saved trajectory bit for bit.  Returns the number of tensors restored."""
    with np.load(path) as z:
        n = int(z["n_tensors"][0])
        for i in range(n):
            numel, step = (int(v) for v in z[f"{i}.meta"])
            opt.set_state(i, dict(numel=numel, step=step, m_codes=z[f"{i}.m_codes"], v_codes=z[f"{i}.v_codes"],
                                  m_scales=z[f"{i}.m_scales"], v_scales=z[f"{i}.v_scales"]))
    return n
