"""GPU parity of QloraLinear forward/backward through the C ABI.

* exact fp32 path: bit-for-bit equal to the CPU oracle (stronger than the reference's own
  GPU-vs-CPU tolerances of 1e-3..1e-2, qlora-wgpu/tests/gpu_parity.rs, gpu_backward.rs);
* tensor-core path (bf16 operands, fp32 accumulate): relative Frobenius error <= 5e-3 vs the
  fp32 oracle evaluated on the same bf16-rounded activations.
"""
import numpy as np
import pytest

from gpu_util import tile_error_report
from refdata import bf16_bits_to_f32, normal, pattern, rel_fro, to_bf16_bits, to_bf16_f32

pytestmark = pytest.mark.gpu
TOL_BF16 = 5e-3  # north-star tolerance for bf16-operand / fp32-accumulate GEMMs


@pytest.fixture(scope="module")
def v():
    import vkqlora.rs_b200 as v

    return v


@pytest.fixture()
def exact_ctx(v):
    ctx = v.GpuContext(0)
    ctx.set_precision(v.PRECISION_FP32_EXACT)
    yield ctx
    ctx.close()


@pytest.fixture()
def tc_ctx(v):
    ctx = v.GpuContext(0)
    ctx.set_precision(v.PRECISION_BF16)
    yield ctx
    ctx.close()


# ---- plain GEMMs: qlora-wgpu/tests/gpu_backward.rs:20-54 ------------------------------------------
def test_gemms_match_cpu_on_odd_sizes_bitwise(v, oracle, exact_ctx):
    m, k, n = 18, 20, 33
    a = pattern(m * k, 11, 13, 13.0, 0.5)
    b_nn, b_nt, b_tn = pattern(k * n, 7, 11, 11.0, 0.5), pattern(n * k, 5, 9, 9.0, 0.5), pattern(m * n, 3, 7, 7.0, 0.5)
    assert np.array_equal(v.gpu_matmul(exact_ctx, a, b_nn, m, k, n), oracle.matmul(a, b_nn, m, k, n))
    assert np.array_equal(v.gpu_matmul_trans_b(exact_ctx, a, b_nt, m, k, n), oracle.matmul_trans_b(a, b_nt, m, k, n))
    assert np.array_equal(v.gpu_matmul_trans_a(exact_ctx, a, b_tn, m, k, n), oracle.matmul_trans_a(a, b_tn, m, k, n))
    # known answer, lora.rs:190-194
    assert v.gpu_matmul(exact_ctx, [1, 2, 3, 4], [5, 6, 7, 8], 2, 2, 2).tolist() == [19.0, 22.0, 43.0, 50.0]
    with pytest.raises(v.ShapeMismatch):
        v.gpu_matmul(exact_ctx, a, b_nn, m, k + 1, n)
    assert v.gpu_matmul(exact_ctx, [], [], 0, 3, 0).size == 0  # kernels.rs:151-153


def _layer_and_oracle(v, oracle, ctx, w, out_dim, in_dim, a=None, b=None, r=0, alpha=0.0, cfg=None):
    cfg = cfg or v.QuantConfig()
    ad = v.LoraAdapter(a, b, in_dim, out_dim, r, alpha) if r else None
    layer = v.QloraLinear.new(w, out_dim, in_dim, cfg, ad, ctx)
    wd = oracle.quantize_nf4(w, out_dim, in_dim, cfg.block_size, cfg.double_quant).dequantize()
    return layer, wd


@pytest.mark.parametrize("out_dim,in_dim,r,batch", [(18, 20, 5, 3), (8, 32, 4, 2), (3, 4, 2, 2), (576, 576, 8, 32), (64, 128, 16, 7)])
def test_exact_path_is_bitwise_equal_to_oracle(v, oracle, exact_ctx, out_dim, in_dim, r, batch):
    w = normal(1, out_dim * in_dim, 0.02)
    a, b = normal(2, r * in_dim, 1.0 / np.sqrt(in_dim)), normal(3, out_dim * r, 0.01)
    x, dy = normal(4, batch * in_dim), normal(5, batch * out_dim)
    alpha = 2.0 * r
    layer, wd = _layer_and_oracle(v, oracle, exact_ctx, w, out_dim, in_dim, a, b, r, alpha)
    y = v.gpu_qlora_forward(exact_ctx, layer, x, batch)
    assert np.array_equal(y, oracle.qlora_forward(x, batch, wd, out_dim, in_dim, a, b, r, alpha)), "forward"
    g = v.gpu_qlora_backward(exact_ctx, layer, x, dy, batch)
    gx, ga, gb = oracle.qlora_backward(x, dy, batch, wd, out_dim, in_dim, a, b, r, alpha)
    assert np.array_equal(g.grad_x, gx), "grad_x"
    assert np.array_equal(g.grad_a, ga), "grad_a"
    assert np.array_equal(g.grad_b, gb), "grad_b"
    # no adapter: grads are None (qlora.rs:139-140)
    layer0, _ = _layer_and_oracle(v, oracle, exact_ctx, w, out_dim, in_dim)
    g0 = layer0.backward(x, dy, batch)
    assert g0.grad_a is None and g0.grad_b is None
    assert np.array_equal(g0.grad_x, oracle.qlora_backward(x, dy, batch, wd, out_dim, in_dim)[0])
    assert np.array_equal(layer0.forward(x, batch), oracle.qlora_forward(x, batch, wd, out_dim, in_dim))


def test_exact_path_other_block_sizes_and_plain_scales(v, oracle, exact_ctx):
    out_dim, in_dim, r, batch = 24, 40, 3, 5
    w = normal(7, out_dim * in_dim, 0.05)
    a, b = normal(8, r * in_dim, 0.2), normal(9, out_dim * r, 0.1)
    x, dy = normal(10, batch * in_dim), normal(11, batch * out_dim)
    for cfg in (v.QuantConfig(32, True), v.QuantConfig(7, False), v.QuantConfig(64, False)):
        layer, wd = _layer_and_oracle(v, oracle, exact_ctx, w, out_dim, in_dim, a, b, r, 6.0, cfg)
        assert np.array_equal(layer.forward(x, batch), oracle.qlora_forward(x, batch, wd, out_dim, in_dim, a, b, r, 6.0))
        g = layer.backward(x, dy, batch)
        gx, ga, gb = oracle.qlora_backward(x, dy, batch, wd, out_dim, in_dim, a, b, r, 6.0)
        assert np.array_equal(g.grad_x, gx) and np.array_equal(g.grad_a, ga) and np.array_equal(g.grad_b, gb)


def test_reference_layer_tests_on_gpu(v, exact_ctx):
    # qlora-core/tests/qlora.rs:13-68 (fused vs unfused fp32, max_err < 0.2)
    out_dim, in_dim, r = 4, 8, 2
    w, a, b = pattern(32, 37, 17, 8.0, 1.0), pattern(16, 13, 7, 7.0, 0.5), pattern(8, 29, 5, 5.0, 0.5)
    x = np.full(2 * in_dim, 0.5, np.float32)
    layer = v.QloraLinear.new(w, out_dim, in_dim, v.QuantConfig(), v.LoraAdapter(a, b, in_dim, out_dim, r, 8.0), exact_ctx)
    y = layer.forward(x, 2).reshape(2, out_dim)
    X, W, A, B = x.reshape(2, in_dim), w.reshape(out_dim, in_dim), a.reshape(r, in_dim), b.reshape(out_dim, r)
    assert np.max(np.abs(y - (X @ W.T + 4.0 * (X @ A.T) @ B.T))) < 0.2
    # :172-198 set_weights changes the forward; wrong sizes are rejected
    b2 = np.full(out_dim * r, 0.5, np.float32)
    layer.adapter_mut().set_weights(a, b2)
    assert not np.array_equal(layer.forward(x, 2).reshape(2, out_dim), y)
    with pytest.raises(v.ShapeMismatch):
        layer.adapter_mut().set_weights([1.0], b2)
    # :200-207 dimension mismatches
    bad = v.LoraAdapter(np.full(16, 0.1, np.float32), np.full(10, 0.1, np.float32), 8, 5, 2, 8.0)
    with pytest.raises(v.ShapeMismatch):
        v.QloraLinear.new(np.full(32, 0.1, np.float32), 4, 8, v.QuantConfig(), bad, exact_ctx)
    ok = v.QloraLinear.new(np.full(32, 0.1, np.float32), 4, 8, v.QuantConfig(), None, exact_ctx)
    with pytest.raises(v.ShapeMismatch):
        ok.forward(np.ones(7, np.float32), 1)
    with pytest.raises(v.ShapeMismatch):
        ok.backward(np.ones(8, np.float32), np.ones(3, np.float32), 1)
    with pytest.raises(v.InvalidConfig):
        v.LoraAdapter([], [], 8, 4, 0, 1.0)


# ---- tensor-core path ------------------------------------------------------------------------------
def _tc_case(v, oracle, ctx, out_dim, in_dim, r, batch, rows_checked=None, cfg=None, seed=0):
    w = normal(1 + seed, out_dim * in_dim, 0.02)
    a = normal(2 + seed, r * in_dim, 1.0 / np.sqrt(in_dim)) if r else None
    b = normal(3 + seed, out_dim * r, 0.01) if r else None
    # activations are bf16 on the device; the oracle consumes the same rounded values as fp32
    x = to_bf16_f32(normal(4 + seed, batch * in_dim))
    dy = to_bf16_f32(normal(5 + seed, batch * out_dim))
    alpha = 2.0 * r
    layer, wd = _layer_and_oracle(v, oracle, ctx, w, out_dim, in_dim, a, b, r, alpha, cfg)
    return layer, wd, x, dy, a, b, alpha


def _assert_close(name, got, want, rows, cols, tol=TOL_BF16):
    err = rel_fro(got, want)
    assert np.all(np.isfinite(got)), f"{name}: non-finite values"
    assert err <= tol, f"{name}: relative Frobenius error {err:.3e} > {tol}\nper-tile relative error:\n" + \
        tile_error_report(got, want, rows, cols)


@pytest.mark.parametrize("out_dim,in_dim,r,batch", [
    (256, 256, 0, 256),     # main GEMM only, one tile
    (256, 256, 16, 256),    # + LoRA extension
    (512, 320, 8, 300),     # ragged rows, several k-steps, two column tiles
    (576, 576, 8, 32),      # benchmark configuration 1 shape: partial column tile, few rows
    (320, 1024, 64, 1000),  # rank 64
    (256, 256, 5, 70),      # the reference GPU test's rank (qlora-wgpu/tests/gpu_backward.rs:60)
    (320, 256, 96, 300),    # ranks above 64: the rank-padded products run in 64-column slices
    (256, 384, 130, 200),   # three slices, the last one nearly empty
    (256, 256, 256, 128),   # the largest rank the tensor-core path takes
])
def test_tensor_core_path_vs_oracle(v, oracle, tc_ctx, out_dim, in_dim, r, batch):
    layer, wd, x, dy, a, b, alpha = _tc_case(v, oracle, tc_ctx, out_dim, in_dim, r, batch)
    y = layer.forward(x, batch)
    _assert_close("forward", y, oracle.qlora_forward(x, batch, wd, out_dim, in_dim, a, b, r, alpha, threads=8), batch, out_dim)
    g = layer.backward(x, dy, batch)
    gx, ga, gb = oracle.qlora_backward(x, dy, batch, wd, out_dim, in_dim, a, b, r, alpha, threads=8)
    _assert_close("grad_x", g.grad_x, gx, batch, in_dim)
    if r:
        _assert_close("grad_a", g.grad_a, ga, r, in_dim)
        _assert_close("grad_b", g.grad_b, gb, out_dim, r)
    else:
        assert g.grad_a is None and g.grad_b is None


@pytest.mark.parametrize("out_dim,in_dim,r,batch,block", [
    (18, 20, 5, 3, 64),       # the reference's own GPU test shape (qlora-wgpu/tests/gpu_backward.rs:56-60)
    (33, 20, 0, 18, 64),      # no adapter; the odd sizes of gpu_backward.rs:20-24
    (100, 200, 96, 70, 64),   # rank above 64 on ragged dimensions
    (130, 70, 128, 257, 64),  # ragged rows as well
    (576, 100, 16, 300, 64),  # only in_dim ragged
    (64, 128, 16, 7, 48),     # aligned dimensions, a block size the fused kernels do not take
    (50, 36, 4, 40, 7),       # everything odd
])
def test_tensor_core_path_ragged_dimensions_and_block_sizes(v, oracle, tc_ctx, out_dim, in_dim, r, batch, block):
    """Dimensions that are no multiple of 64 and arbitrary block sizes stay on the tensor cores (the context is
    pinned to them, so a refusal would raise): the layer runs through a zero-padded bf16 copy of itself."""
    layer, wd, x, dy, a, b, alpha = _tc_case(v, oracle, tc_ctx, out_dim, in_dim, r, batch, cfg=v.QuantConfig(block, True),
                                             seed=out_dim + in_dim)
    for _ in range(2):  # the second pass reuses the padded copy
        y = layer.forward(x, batch)
        _assert_close("forward", y, oracle.qlora_forward(x, batch, wd, out_dim, in_dim, a, b, r, alpha, threads=8), batch, out_dim)
        g = layer.backward(x, dy, batch)
        gx, ga, gb = oracle.qlora_backward(x, dy, batch, wd, out_dim, in_dim, a, b, r, alpha, threads=8)
        _assert_close("grad_x", g.grad_x, gx, batch, in_dim)
        if r:
            _assert_close("grad_a", g.grad_a, ga, r, in_dim)
            _assert_close("grad_b", g.grad_b, gb, out_dim, r)
        else:
            assert g.grad_a is None and g.grad_b is None


def test_ragged_layer_follows_adapter_updates_and_slab_accumulation(v, oracle, tc_ctx):
    """A ragged layer's padded copy follows set_adapter_weights, and the slab pipeline of the host entry points
    (gradients summed slab after slab) gives the gradients of the whole batch."""
    from vkqlora.rs_b200 import _lib
    out_dim, in_dim, r, batch = 100, 200, 8, 2 * 2048 + 300
    layer, wd, x, dy, a, b, alpha = _tc_case(v, oracle, tc_ctx, out_dim, in_dim, r, batch, seed=77)
    layer.forward(x[:in_dim * 4], 4)  # builds the padded copy with the first adapter
    a2, b2 = normal(91, r * in_dim, 0.05), normal(92, out_dim * r, 0.05)
    layer.adapter_mut().set_weights(a2, b2)
    xb, dyb = to_bf16_bits(x), to_bf16_bits(dy)
    y = bf16_bits_to_f32(layer.forward_host(xb, batch, v.DTYPE_BF16))
    _assert_close("forward", y, oracle.qlora_forward(x, batch, wd, out_dim, in_dim, a2, b2, r, alpha, threads=8), batch, out_dim,
                  tol=6e-3)  # + the bf16 rounding of the returned Y
    gx = np.empty(batch * in_dim, np.uint16)
    ga, gb = np.empty(r * in_dim, np.float32), np.empty(out_dim * r, np.float32)
    _lib.check(_lib.lib.qlc_qlora_backward_host(tc_ctx._h, layer._h, xb.ctypes.data, dyb.ctypes.data, v.DTYPE_BF16, batch,
                                                gx.ctypes.data, ga.ctypes.data, gb.ctypes.data))
    gx_ref, ga_ref, gb_ref = oracle.qlora_backward(x, dy, batch, wd, out_dim, in_dim, a2, b2, r, alpha, threads=8)
    _assert_close("grad_x", bf16_bits_to_f32(gx), gx_ref, batch, in_dim, tol=6e-3)
    _assert_close("grad_a", ga, ga_ref, r, in_dim)
    _assert_close("grad_b", gb, gb_ref, out_dim, r)


def test_tensor_core_path_plain_fp32_scales(v, oracle, tc_ctx):
    # from_raw_parts tensors carry fp32 scales (what the Python entry points rebuild)
    layer, wd, x, dy, a, b, alpha = _tc_case(v, oracle, tc_ctx, 256, 384, 16, 128, cfg=v.QuantConfig(64, False))
    _assert_close("forward", layer.forward(x, 128), oracle.qlora_forward(x, 128, wd, 256, 384, a, b, 16, alpha, threads=8), 128, 256)


@pytest.mark.parametrize("block_size", [32, 128, 256])
@pytest.mark.parametrize("double_quant", [True, False])
def test_tensor_core_path_other_block_sizes(v, oracle, tc_ctx, block_size, double_quant):
    """Quantisation blocks of 32, 128 and 256 elements on the tensor-core path (the context is pinned to it, so an
    ineligible layer would raise instead of falling back).  in_dim = 320 is no multiple of 128 or 256: blocks
    straddle weight rows, as the flat blocking of quant.rs:100-118 allows."""
    out_dim, in_dim, r, batch = 512, 320, 8, 300
    layer, wd, x, dy, a, b, alpha = _tc_case(v, oracle, tc_ctx, out_dim, in_dim, r, batch,
                                             cfg=v.QuantConfig(block_size, double_quant), seed=block_size)
    _assert_close("forward", layer.forward(x, batch),
                  oracle.qlora_forward(x, batch, wd, out_dim, in_dim, a, b, r, alpha, threads=8), batch, out_dim)
    g = layer.backward(x, dy, batch)
    gx, ga, gb = oracle.qlora_backward(x, dy, batch, wd, out_dim, in_dim, a, b, r, alpha, threads=8)
    _assert_close("grad_x", g.grad_x, gx, batch, in_dim)
    _assert_close("grad_a", g.grad_a, ga, r, in_dim)
    _assert_close("grad_b", g.grad_b, gb, out_dim, r)


def test_tensor_core_full_size_4096_sampled_rows(v, oracle, tc_ctx):
    """benchmark configuration 2 (4096x4096, 8192 rows, r=16, alpha=32) through the host bf16 entry point.
    Rows of Y and dX are independent, so a seeded sample of rows (plus tile-edge rows) is compared
    with the oracle; grad_A / grad_B contract over all rows and are compared in full."""
    out_dim = in_dim = 4096
    batch, r, alpha = 8192, 16, 32.0
    w = normal(1, out_dim * in_dim, 0.02)
    a, b = normal(2, r * in_dim, 1.0 / 64.0), normal(3, out_dim * r, 0.01)
    xb, dyb = to_bf16_bits(normal(4, batch * in_dim)), to_bf16_bits(normal(5, batch * out_dim))
    layer, wd = _layer_and_oracle(v, oracle, tc_ctx, w, out_dim, in_dim, a, b, r, alpha)
    import ctypes as C
    from vkqlora.rs_b200 import _lib
    y = layer.forward_host(xb, batch, v.DTYPE_BF16)
    gx = np.empty(batch * in_dim, np.uint16)
    ga, gb = np.empty(r * in_dim, np.float32), np.empty(out_dim * r, np.float32)
    _lib.check(_lib.lib.qlc_qlora_backward_host(tc_ctx._h, layer._h, xb.ctypes.data, dyb.ctypes.data, v.DTYPE_BF16, batch,
                                                gx.ctypes.data, ga.ctypes.data, gb.ctypes.data))
    rng = np.random.default_rng(0)
    rows = np.unique(np.concatenate([[0, 127, 128, 255, 256, 4095, 4096, 8191], rng.integers(0, batch, 40)]))
    xs = bf16_bits_to_f32(xb).reshape(batch, in_dim)[rows].reshape(-1)
    dys = bf16_bits_to_f32(dyb).reshape(batch, out_dim)[rows].reshape(-1)
    y_ref = oracle.qlora_forward(xs, rows.size, wd, out_dim, in_dim, a, b, r, alpha, threads=8)
    _assert_close("forward", bf16_bits_to_f32(y).reshape(batch, out_dim)[rows], y_ref, rows.size, out_dim)
    gx_ref = oracle.qlora_backward(xs, dys, rows.size, wd, out_dim, in_dim, a, b, r, alpha, threads=8)[0]
    _assert_close("grad_x", bf16_bits_to_f32(gx).reshape(batch, in_dim)[rows], gx_ref, rows.size, in_dim)
    # token-contracted gradients in float64 numpy (the oracle's scalar loops would take minutes)
    X = bf16_bits_to_f32(xb).reshape(batch, in_dim).astype(np.float64)
    DY = bf16_bits_to_f32(dyb).reshape(batch, out_dim).astype(np.float64)
    A, B = a.reshape(r, in_dim).astype(np.float64), b.reshape(out_dim, r).astype(np.float64)
    s = alpha / r
    _assert_close("grad_a", ga, ((s * DY) @ B).T @ X, r, in_dim)
    _assert_close("grad_b", gb, (s * DY).T @ (X @ A.T), out_dim, r)


@pytest.mark.parametrize("batch", [2 * 2048 + 300, 5120 + 300])
def test_host_entry_points_pipelined_slabs_match_single_device_call(v, oracle, tc_ctx, batch):
    """The bf16 host entry points split large batches into row slabs that overlap copies and compute: equal
    slabs with a ragged last one (4396 rows), or, from 5120 rows on, slabs that ramp up and down at the ends
    (5420 rows: 512, 1024, 2048, 300, 1024, 512).
    Y and dX rows do not depend on the split (bit-identical to one device call over all rows);
    grad_A / grad_B are summed slab after slab in fp32, so they agree to fp32 rounding."""
    import torch
    from vkqlora.rs_b200 import _lib
    out_dim, in_dim, r = 320, 256, 8
    layer, wd, x, dy, a, b, alpha = _tc_case(v, oracle, tc_ctx, out_dim, in_dim, r, batch, seed=40)
    xb, dyb = to_bf16_bits(x), to_bf16_bits(dy)
    y = layer.forward_host(xb, batch, v.DTYPE_BF16)
    gx = np.empty(batch * in_dim, np.uint16)
    ga, gb = np.empty(r * in_dim, np.float32), np.empty(out_dim * r, np.float32)
    _lib.check(_lib.lib.qlc_qlora_backward_host(tc_ctx._h, layer._h, xb.ctypes.data, dyb.ctypes.data, v.DTYPE_BF16, batch,
                                                gx.ctypes.data, ga.ctypes.data, gb.ctypes.data))
    dev = torch.device("cuda:0")
    tx = torch.from_numpy(xb.view(np.int16)).to(dev)
    tdy = torch.from_numpy(dyb.view(np.int16)).to(dev)
    ty = torch.empty(batch * out_dim, dtype=torch.int16, device=dev)
    tgx = torch.empty(batch * in_dim, dtype=torch.int16, device=dev)
    tga = torch.empty(r * in_dim, dtype=torch.float32, device=dev)
    tgb = torch.empty(out_dim * r, dtype=torch.float32, device=dev)
    torch.cuda.synchronize()
    layer.forward_dev(tx.data_ptr(), batch, ty.data_ptr(), v.DTYPE_BF16)
    layer.backward_dev(tx.data_ptr(), tdy.data_ptr(), batch, tgx.data_ptr(), tga.data_ptr(), tgb.data_ptr(), v.DTYPE_BF16)
    tc_ctx.synchronize()
    assert np.array_equal(y.view(np.int16), ty.cpu().numpy())
    assert np.array_equal(gx.view(np.int16), tgx.cpu().numpy())
    assert rel_fro(ga, tga.cpu().numpy()) <= 1e-5 and rel_fro(gb, tgb.cpu().numpy()) <= 1e-5
    gx_ref, ga_ref, gb_ref = oracle.qlora_backward(x, dy, batch, wd, out_dim, in_dim, a, b, r, alpha, threads=8)
    _assert_close("grad_a", ga, ga_ref, r, in_dim)
    _assert_close("grad_b", gb, gb_ref, out_dim, r)


@pytest.mark.parametrize("batch", [700, 5120 + 300])
def test_fused_forward_backward_host_equals_the_two_stateless_calls(v, oracle, tc_ctx, batch):
    """qlc_qlora_forward_backward_host uploads X once and runs forward and backward slab by slab in one pipeline
    (5420 rows), or falls back to the two calls (700 rows: below the slab threshold).  Y and dX must be
    bit-identical to qlc_qlora_forward_host + qlc_qlora_backward_host; grad_A / grad_B (fp32 sums over slabs in the
    same order) as well; and everything agrees with the oracle."""
    from vkqlora.rs_b200 import _lib
    out_dim, in_dim, r = 320, 256, 8
    layer, wd, x, dy, a, b, alpha = _tc_case(v, oracle, tc_ctx, out_dim, in_dim, r, batch, seed=44)
    xb, dyb = to_bf16_bits(x), to_bf16_bits(dy)
    y2 = layer.forward_host(xb, batch, v.DTYPE_BF16)
    gx2 = np.empty(batch * in_dim, np.uint16)
    ga2, gb2 = np.empty(r * in_dim, np.float32), np.empty(out_dim * r, np.float32)
    _lib.check(_lib.lib.qlc_qlora_backward_host(tc_ctx._h, layer._h, xb.ctypes.data, dyb.ctypes.data, v.DTYPE_BF16, batch,
                                                gx2.ctypes.data, ga2.ctypes.data, gb2.ctypes.data))
    y1, g1 = layer.forward_backward_host(xb, dyb, batch, v.DTYPE_BF16)
    assert np.array_equal(y1, y2) and np.array_equal(g1.grad_x, gx2)
    assert np.array_equal(g1.grad_a, ga2) and np.array_equal(g1.grad_b, gb2)
    y_ref = oracle.qlora_forward(x, batch, wd, out_dim, in_dim, a, b, r, alpha, threads=8)
    gx_ref, ga_ref, gb_ref = oracle.qlora_backward(x, dy, batch, wd, out_dim, in_dim, a, b, r, alpha, threads=8)
    _assert_close("forward", bf16_bits_to_f32(y1), y_ref, batch, out_dim)
    _assert_close("grad_x", bf16_bits_to_f32(g1.grad_x), gx_ref, batch, in_dim)
    _assert_close("grad_a", g1.grad_a, ga_ref, r, in_dim)
    _assert_close("grad_b", g1.grad_b, gb_ref, out_dim, r)
    # gradients may stay on the device (NULL host pointers): the layer's bucket then holds them
    y3, gx3 = np.empty_like(y1), np.empty_like(gx2)
    _lib.check(_lib.lib.qlc_qlora_forward_backward_host(tc_ctx._h, layer._h, xb.ctypes.data, dyb.ctypes.data, v.DTYPE_BF16,
                                                        batch, y3.ctypes.data, gx3.ctypes.data, None, None))
    ptr, n = layer.grad_bucket()
    assert n == r * (in_dim + out_dim)
    got = np.empty(n, np.float32)
    tc_ctx.copy_to_host(got.ctypes.data, ptr, 4 * n)
    tc_ctx.synchronize()
    assert np.array_equal(got[:r * in_dim], ga2) and np.array_equal(got[r * in_dim:], gb2)
    assert np.array_equal(y3, y1) and np.array_equal(gx3, gx2)


def test_async_fused_host_calls_two_in_flight(v, oracle, tc_ctx):
    """qlc_qlora_forward_backward_host_async: three submissions with different inputs, two in flight at a time
    (each with its own pinned host buffers), waited for by ticket.  Every result equals the synchronous call's:
    a submission must not overwrite staged inputs or outputs that an earlier one still needs."""
    import torch
    out_dim, in_dim, r, batch = 320, 256, 8, 5120 + 300
    layer, wd, x0, dy0, a, b, alpha = _tc_case(v, oracle, tc_ctx, out_dim, in_dim, r, batch, seed=46)
    cases = []
    for i in range(3):
        x, dy = to_bf16_bits(normal(460 + i, batch * in_dim)), to_bf16_bits(normal(470 + i, batch * out_dim))
        y, g = layer.forward_backward_host(x, dy, batch, v.DTYPE_BF16)
        cases.append((x, dy, y, g))
    pin = lambda n, dt: torch.empty(n, dtype=dt).pin_memory()
    sets = [dict(x=pin(batch * in_dim, torch.int16), dy=pin(batch * out_dim, torch.int16), y=pin(batch * out_dim, torch.int16),
                 gx=pin(batch * in_dim, torch.int16), ga=pin(r * in_dim, torch.float32), gb=pin(out_dim * r, torch.float32))
            for _ in range(2)]
    tickets, results = [None, None], []

    def collect(k, i):
        tc_ctx.wait(tickets[k])
        s = sets[k]
        results.append((i, s["y"].numpy().copy().view(np.uint16), s["gx"].numpy().copy().view(np.uint16),
                        s["ga"].numpy().copy(), s["gb"].numpy().copy()))

    for i, (x, dy, _, _) in enumerate(cases):
        k = i & 1
        if tickets[k] is not None:
            collect(k, i - 2)
        s = sets[k]
        s["x"].numpy()[:] = x.view(np.int16)
        s["dy"].numpy()[:] = dy.view(np.int16)
        tickets[k] = layer.forward_backward_host_async(s["x"].data_ptr(), s["dy"].data_ptr(), batch, v.DTYPE_BF16,
                                                       s["y"].data_ptr(), s["gx"].data_ptr(), s["ga"].data_ptr(),
                                                       s["gb"].data_ptr())
    collect(1, 1)
    collect(0, 2)
    tc_ctx.synchronize()
    assert sorted(i for i, *_ in results) == [0, 1, 2]
    for i, y, gx, ga, gb in results:
        _, _, y_ref, g_ref = cases[i]
        assert np.array_equal(y, y_ref) and np.array_equal(gx, g_ref.grad_x), i
        # the asynchronous call splits the batch into equal slabs, the synchronous one ramps them: grad_A / grad_B are
        # summed slab after slab in fp32, so the two agree to fp32 rounding
        assert rel_fro(ga, g_ref.grad_a) <= 1e-5 and rel_fro(gb, g_ref.grad_b) <= 1e-5, i
    with pytest.raises(v.InvalidConfig):
        tc_ctx.wait(10**6)


@pytest.mark.parametrize("out_dim,in_dim", [(11008, 4096), (4096, 11008)])
def test_tensor_core_projection_stack_shapes_rank64(v, oracle, tc_ctx, out_dim, in_dim):
    """benchmark configuration 5 shapes (gate/up 11008x4096, down 4096x11008; r=64, alpha=128): 43 column tiles
    (not a multiple of anything convenient), a ragged last row tile, cut tiles in the last wave.
    Sampled rows of Y / dX against the oracle; grad_A / grad_B in full against float64 numpy."""
    batch, r, alpha = 1000, 64, 128.0
    w = normal(11, out_dim * in_dim, 0.02)
    a, b = normal(12, r * in_dim, 1.0 / np.sqrt(in_dim)), normal(13, out_dim * r, 0.01)
    x, dy = to_bf16_f32(normal(14, batch * in_dim)), to_bf16_f32(normal(15, batch * out_dim))
    layer, wd = _layer_and_oracle(v, oracle, tc_ctx, w, out_dim, in_dim, a, b, r, alpha)
    y = layer.forward(x, batch)
    g = layer.backward(x, dy, batch)
    rows = np.unique(np.concatenate([[0, 127, 128, 511, 512, 999], np.random.default_rng(1).integers(0, batch, 10)]))
    xs = x.reshape(batch, in_dim)[rows].reshape(-1)
    dys = dy.reshape(batch, out_dim)[rows].reshape(-1)
    _assert_close("forward", y.reshape(batch, out_dim)[rows],
                  oracle.qlora_forward(xs, rows.size, wd, out_dim, in_dim, a, b, r, alpha, threads=8), rows.size, out_dim)
    gx_ref = oracle.qlora_backward(xs, dys, rows.size, wd, out_dim, in_dim, a, b, r, alpha, threads=8)[0]
    _assert_close("grad_x", g.grad_x.reshape(batch, in_dim)[rows], gx_ref, rows.size, in_dim)
    X, DY = x.reshape(batch, in_dim).astype(np.float64), dy.reshape(batch, out_dim).astype(np.float64)
    A, B = a.reshape(r, in_dim).astype(np.float64), b.reshape(out_dim, r).astype(np.float64)
    s = alpha / r
    _assert_close("grad_a", g.grad_a, ((s * DY) @ B).T @ X, r, in_dim)
    _assert_close("grad_b", g.grad_b, (s * DY).T @ (X @ A.T), out_dim, r)


# ---- TF32 mode ---------------------------------------------------------------------------------------
TOL_TF32 = 1e-3  # relative Frobenius error vs the fp32 oracle (north-star tolerance of the TF32 mode)


@pytest.fixture()
def tf32_ctx(v):
    ctx = v.GpuContext(0)
    ctx.set_precision(v.PRECISION_TF32)
    yield ctx
    ctx.close()


@pytest.mark.parametrize("out_dim,in_dim,r,batch", [
    (256, 256, 0, 256),     # weight GEMM only
    (256, 256, 16, 256),    # + LoRA (rank 16: narrow side products)
    (512, 320, 8, 300),     # ragged rows, several k-steps, two column tiles
    (576, 576, 8, 32),      # benchmark configuration 1 shape
    (320, 1024, 64, 1000),  # rank 64, cut tiles
    (320, 256, 96, 300),    # rank above 64 (two 64-column slices)
])
def test_tf32_mode_vs_oracle(v, oracle, tf32_ctx, out_dim, in_dim, r, batch):
    _tf32_case(v, oracle, tf32_ctx, out_dim, in_dim, r, batch, None)


@pytest.mark.parametrize("block_size", [32, 256])
def test_tf32_mode_other_block_sizes(v, oracle, tf32_ctx, block_size):
    _tf32_case(v, oracle, tf32_ctx, 512, 320, 8, 300, v.QuantConfig(block_size, True))


def _tf32_case(v, oracle, tf32_ctx, out_dim, in_dim, r, batch, cfg):
    """fp32 activations that are NOT bf16-representable: the tensor core truncates them to tf32."""
    w = normal(21, out_dim * in_dim, 0.02)
    a = normal(22, r * in_dim, 1.0 / np.sqrt(in_dim)) if r else None
    b = normal(23, out_dim * r, 0.01) if r else None
    x, dy = normal(24, batch * in_dim), normal(25, batch * out_dim)
    alpha = 2.0 * r
    layer, wd = _layer_and_oracle(v, oracle, tf32_ctx, w, out_dim, in_dim, a, b, r, alpha, cfg)
    y = layer.forward(x, batch)
    _assert_close("forward", y, oracle.qlora_forward(x, batch, wd, out_dim, in_dim, a, b, r, alpha, threads=8), batch, out_dim,
                  tol=TOL_TF32)
    g = layer.backward(x, dy, batch)
    gx, ga, gb = oracle.qlora_backward(x, dy, batch, wd, out_dim, in_dim, a, b, r, alpha, threads=8)
    _assert_close("grad_x", g.grad_x, gx, batch, in_dim, tol=TOL_TF32)
    if r:
        _assert_close("grad_a", g.grad_a, ga, r, in_dim, tol=TOL_TF32)
        _assert_close("grad_b", g.grad_b, gb, out_dim, r, tol=TOL_TF32)


def test_reserved_sms_leave_results_unchanged(v, oracle, tc_ctx):
    """qlc_ctx_set_reserved_sms only changes how many CTA pairs walk the tile list of the weight GEMMs: the results of
    a shape with several tiles per pair are bit-identical with 0, 4 and 40 SMs reserved; bad values are refused."""
    out_dim, in_dim, r, batch = 1024, 512, 16, 9000   # 18 row tiles x 4 column tiles = 72 tiles, k-cut candidates
    layer, wd, x, dy, a, b, alpha = _tc_case(v, oracle, tc_ctx, out_dim, in_dim, r, batch, seed=61)
    results = []
    for sms in (0, 4, 40):
        tc_ctx.set_reserved_sms(sms)
        y = layer.forward(x, batch)
        g = layer.backward(x, dy, batch)
        results.append((y, g.grad_x))
    tc_ctx.set_reserved_sms(0)
    for y, gx in results[1:]:
        # (tiles cut along the contraction are summed in chunk order whatever the pair count: still bit-identical
        #  unless the cut plan itself changes with the pair count, hence the tolerance on top of exact equality)
        assert np.array_equal(y, results[0][0]) or rel_fro(y, results[0][0]) <= 1e-6
        assert np.array_equal(gx, results[0][1]) or rel_fro(gx, results[0][1]) <= 1e-6
    _assert_close("forward", results[1][0], oracle.qlora_forward(x, batch, wd, out_dim, in_dim, a, b, r, alpha, threads=8), batch, out_dim)
    with pytest.raises(v.InvalidConfig):
        tc_ctx.set_reserved_sms(-2)
    with pytest.raises(v.InvalidConfig):
        tc_ctx.set_reserved_sms(10**6)
