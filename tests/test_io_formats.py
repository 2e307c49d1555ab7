"""On-disk formats: safetensors header rules (qlora-io/src/safetensors.rs:25-76), widening of stored
dtypes (:82-99), stored-npz adapters (qlora-io/src/npz.rs:46-104, tools/npz2pt.py:28-32), and - on the
GPU - quantising a checkpoint tensor from its stored dtype with codes equal to the oracle's."""
import json
import struct
import zipfile

import numpy as np
import pytest

from refdata import normal


@pytest.fixture(scope="module")
def io():
    from vkqlora.rs_b200 import io

    return io


def _bf16_bits(x):
    u = np.ascontiguousarray(x, np.float32).view(np.uint32).astype(np.uint64)
    return ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)


def test_safetensors_round_trip_and_widening(io, tmp_path):
    w32 = normal(1, 6 * 8, 0.02).reshape(6, 8)
    w16 = w32.astype(np.float16)
    wbf = _bf16_bits(w32).reshape(6, 8)
    p = str(tmp_path / "m.safetensors")
    io.write_safetensors(p, {"a.weight": w32, "b.weight": w16, "c.weight": ("BF16", wbf)})
    with io.SafetensorsFile(p) as f:
        assert set(f.names()) == {"a.weight", "b.weight", "c.weight"}
        assert f.entries["c.weight"][:2] == ("BF16", (6, 8))
        assert np.array_equal(f.to_f32("a.weight"), w32)
        assert np.array_equal(f.to_f32("b.weight"), w16.astype(np.float32))
        assert np.array_equal(f.to_f32("c.weight").view(np.uint32), wbf.astype(np.uint32) << 16)


def _write_raw(path, header: dict, data: bytes, hlen_override=None):
    hj = json.dumps(header).encode()
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(hj) if hlen_override is None else hlen_override))
        f.write(hj)
        f.write(data)


def test_safetensors_malformed_files_are_rejected(io, tmp_path):
    import vkqlora.rs_b200 as v
    p = str(tmp_path / "bad.safetensors")
    open(p, "wb").write(b"abc")                                     # smaller than the header length field
    with pytest.raises(v.InvalidConfig):
        io.SafetensorsFile(p)
    _write_raw(p, {}, b"", hlen_override=10_000)                      # header length exceeds file
    with pytest.raises(v.InvalidConfig):
        io.SafetensorsFile(p)
    _write_raw(p, {"w": {"dtype": "F32", "shape": [2, 2], "data_offsets": [0, 64]}}, b"\0" * 16)   # outside data
    with pytest.raises(v.InvalidConfig):
        io.SafetensorsFile(p)
    _write_raw(p, {"w": {"dtype": "F32", "shape": [2, 3], "data_offsets": [0, 16]}}, b"\0" * 16)   # size mismatch
    with pytest.raises(v.ShapeMismatch):
        io.SafetensorsFile(p)
    _write_raw(p, {"w": {"dtype": "F8_E4M3", "shape": [4], "data_offsets": [0, 4]}}, b"\0" * 4)    # unsupported
    with pytest.raises(v.InvalidConfig):
        io.SafetensorsFile(p)


def test_adapters_npz_is_stored_f4_and_round_trips(io, tmp_path):
    a, b = normal(2, 4 * 16, 0.1).reshape(4, 16), normal(3, 8 * 4, 0.1).reshape(8, 4)
    p = str(tmp_path / "adapters.npz")
    io.save_adapters_npz(p, {"layers.0.q_proj.lora_A": a, "layers.0.q_proj.lora_B": b.astype(np.float64)})
    with zipfile.ZipFile(p) as z:
        assert all(i.compress_type == zipfile.ZIP_STORED for i in z.infolist())
        assert sorted(z.namelist()) == ["layers.0.q_proj.lora_A.npy", "layers.0.q_proj.lora_B.npy"]
    with np.load(p) as z:                       # what tools/npz2pt.py does
        assert z["layers.0.q_proj.lora_A"].dtype == np.dtype("<f4")
        assert np.array_equal(z["layers.0.q_proj.lora_A"], a)
    back = io.load_adapters_npz(p)
    assert np.array_equal(back["layers.0.q_proj.lora_B"], b)


@pytest.mark.gpu
@pytest.mark.parametrize("stored", ["F32", "BF16", "F16"])
def test_quantize_from_checkpoint_dtype_is_bit_exact(io, oracle, tmp_path, stored):
    import vkqlora.rs_b200 as v
    rows, cols = 96, 200   # blocks straddle rows, ragged last block
    w32 = normal(4, rows * cols, 0.02).reshape(rows, cols)
    if stored == "F32":
        tensor, widened = w32, w32
    elif stored == "F16":
        tensor = w32.astype(np.float16)
        widened = tensor.astype(np.float32)
    else:
        bits = _bf16_bits(w32).reshape(rows, cols)
        tensor = ("BF16", bits)
        widened = (bits.astype(np.uint32) << 16).view(np.float32)
    p = str(tmp_path / "ckpt.safetensors")
    io.write_safetensors(p, {"model.layers.0.self_attn.q_proj.weight": tensor})
    ctx = v.GpuContext(0)
    with io.SafetensorsFile(p) as f:
        q = f.quantize("model.layers.0.self_attn.q_proj.weight", v.QuantConfig(), ctx)
    ref = oracle.quantize_nf4(np.ascontiguousarray(widened).reshape(-1), rows, cols)
    assert np.array_equal(q.codes(), ref.codes)
    assert np.array_equal(q.absmax_codes(), ref.absmax_codes)
    assert np.array_equal(q.absmax2().view(np.uint32), ref.absmax2.view(np.uint32))


@pytest.mark.gpu
def test_persisted_nf4_payload_and_adam_state_round_trip(io, oracle, tmp_path):
    """A quantised tensor saved with save_quantized_npz comes back bit for bit without a quantisation pass (double
    quantised and plain-scale forms), and a saved optimiser state continues the trajectory bit for bit."""
    import vkqlora.rs_b200 as v
    ctx = v.GpuContext(0)
    rows, cols = 96, 200
    w = normal(11, rows * cols, 0.02)
    qd = v.QuantizedTensor.quantize(w, rows, cols, v.QuantConfig(64, True), ctx)
    qf = v.QuantizedTensor.quantize(w, rows, cols, v.QuantConfig(32, False), ctx)
    p = str(tmp_path / "payload.npz")
    io.save_quantized_npz(p, {"layers.0.q_proj": qd, "layers.0.v_proj": qf})
    with zipfile.ZipFile(p) as z:
        assert all(i.compress_type == zipfile.ZIP_STORED for i in z.infolist())
    back = io.load_quantized_npz(p, ctx)
    assert sorted(back) == ["layers.0.q_proj", "layers.0.v_proj"]
    bd, bf = back["layers.0.q_proj"], back["layers.0.v_proj"]
    assert bd.uses_double_quant() and not bf.uses_double_quant()
    assert (bd.rows(), bd.cols(), bd.block_size()) == (rows, cols, 64) and bf.block_size() == 32
    assert np.array_equal(bd.codes(), qd.codes()) and np.array_equal(bd.absmax_codes(), qd.absmax_codes())
    assert np.array_equal(bd.absmax2().view(np.uint32), qd.absmax2().view(np.uint32))
    assert np.array_equal(bd.dequantize().view(np.uint32), qd.dequantize().view(np.uint32))
    assert np.array_equal(bf.codes(), qf.codes())
    assert np.array_equal(bf.dequantize().view(np.uint32), qf.dequantize().view(np.uint32))
    ref = oracle.quantize_nf4(w, rows, cols)
    assert np.array_equal(bd.dequantize().view(np.uint32), ref.dequantize().view(np.uint32))

    sizes = [1000, 4096 + 13]
    a = v.Adam8bit(v.AdamConfig(), ctx)
    pa = [normal(30 + i, n, 0.01) for i, n in enumerate(sizes)]
    for t in range(2):
        a.step(pa, [normal(500 * t + i, n, 0.01) for i, n in enumerate(sizes)])
    ps = str(tmp_path / "adam.npz")
    io.save_adam_state_npz(ps, a, len(sizes))
    b = v.Adam8bit(v.AdamConfig(max_resident_pages=1), ctx)  # restored into a paged optimiser
    assert io.load_adam_state_npz(ps, b) == len(sizes)
    pb = [x.copy() for x in pa]
    g = [normal(900 + i, n, 0.01) for i, n in enumerate(sizes)]
    a.step(pa, g)
    b.step(pb, g)
    for i in range(len(sizes)):
        assert np.array_equal(pa[i].view(np.uint32), pb[i].view(np.uint32))
        sa, sb = a.get_state(i), b.get_state(i)
        assert sa["step"] == sb["step"] == 3
        for k in ("m_codes", "v_codes", "m_scales", "v_scales"):
            assert np.array_equal(sa[k], sb[k]), (i, k)
