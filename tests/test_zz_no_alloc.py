"""The allocation-free forward entry point (qlc_qlora_forward_dev_noalloc), tested last.

It exists for hosts that cannot let the library call cudaMalloc while they run (all spare device memory
already handed to their own pool; step loops that cannot take the device-wide stall of a driver
allocation).  Its scratch is one fixed array shared by every call on the device, so:

  * it must give the result of the regular device entry point (qlc_qlora_forward_dev) call after call - a
    large batch, then a smaller one with other data: stale rows of the first call must not leak into the second;
  * it must really allocate nothing: on a context that never ran the regular path (whose scratch arena is
    therefore still empty), free device memory is the same before and after, at the entry point's largest
    batch (8192 rows);
  * one row more is refused with a message that names the limit.
The file name sorts last on purpose: if this addition ever breaks, every other test has already run.
"""
import numpy as np
import pytest

from refdata import rel_fro

pytestmark = pytest.mark.gpu


def _layer(v, ctx, out_dim, in_dim, r, alpha, seed):
    g = np.random.Generator(np.random.Philox(seed))
    w = (g.standard_normal(out_dim * in_dim) * 0.02).astype(np.float32)
    a = (g.standard_normal(r * in_dim) / np.sqrt(in_dim)).astype(np.float32)
    b = (g.standard_normal(out_dim * r) * 0.01).astype(np.float32)
    layer = v.QloraLinear.new(w, out_dim, in_dim, v.QuantConfig(), v.LoraAdapter(a, b, in_dim, out_dim, r, alpha), ctx)
    return layer, w, a, b


def test_noalloc_forward_matches_regular_forward_twice(oracle):
    import torch

    import vkqlora.rs_b200 as v
    from vkqlora.rs_b200 import _lib

    dev = torch.device("cuda", 0)
    out_dim, in_dim, r, alpha = 512, 384, 16, 32.0
    ctx_new = v.GpuContext(0)   # only ever runs the allocation-free entry point
    ctx_ref = v.GpuContext(0)   # the regular entry point, on a context of its own
    layer_new, w, a, b = _layer(v, ctx_new, out_dim, in_dim, r, alpha, 42)
    layer_ref, _, _, _ = _layer(v, ctx_ref, out_dim, in_dim, r, alpha, 42)
    wd = oracle.quantize_nf4(w, out_dim, in_dim).dequantize()

    gen = torch.Generator(device=dev).manual_seed(7)
    for batch in (1000, 300):  # two calls in a row; the second reuses the scratch rows of the first
        x = torch.randn(batch, in_dim, generator=gen, device=dev).to(torch.bfloat16)
        y_ref = torch.empty(batch, out_dim, device=dev, dtype=torch.bfloat16)
        y_new = torch.zeros(batch, out_dim, device=dev, dtype=torch.bfloat16)
        torch.cuda.synchronize()
        layer_ref.forward_dev(x.data_ptr(), batch, y_ref.data_ptr(), v.DTYPE_BF16)   # existing entry point
        ctx_ref.synchronize()
        layer_new.forward_dev_noalloc(x.data_ptr(), batch, y_new.data_ptr())          # new entry point
        ctx_new.synchronize()
        ref = y_ref.float().cpu().numpy()
        new = y_new.float().cpu().numpy()
        assert np.all(np.isfinite(new))
        # same kernels, same inputs: the tolerance of the other tensor-core tests (5e-3 relative
        # Frobenius) is the bar; at these sizes neither path cuts tiles and the two results are identical
        assert rel_fro(new, ref) <= 5e-3, batch
        assert np.array_equal(new, ref), batch
        # ... and both agree with the CPU oracle on the same bf16 inputs
        want = oracle.qlora_forward(x.float().cpu().numpy().reshape(-1), batch, wd, out_dim, in_dim, a, b, r, alpha)
        assert rel_fro(new, want) <= 5e-3, batch

    # sizes beyond the fixed scratch are refused with a clear message, not truncated
    big = 8193
    x = torch.zeros(big, in_dim, device=dev, dtype=torch.bfloat16)
    y = torch.zeros(big, out_dim, device=dev, dtype=torch.bfloat16)
    with pytest.raises(v.InvalidConfig) as e:
        layer_new.forward_dev_noalloc(x.data_ptr(), big, y.data_ptr())
    assert "8192" in str(e.value)
    assert hasattr(_lib.lib, "qlc_qlora_forward_dev_noalloc")


def test_noalloc_forward_allocates_nothing_at_its_largest_batch(oracle):
    """8192 rows of a 4096x4096 layer (the headline benchmark shape) on a fresh context: free device memory does
    not move across the calls (the regular entry point grows the context's scratch arena by tens of MiB here),
    and the result agrees with the regular entry point.  At this size the regular path cuts the tiles of its
    last wave along the contraction and adds fp32 partials, which the allocation-free path (no scratch for
    partials) does not: the two may differ in the last bf16 bit, so the comparison uses the tensor-core
    tolerance (5e-3 relative Frobenius)."""
    import torch

    import vkqlora.rs_b200 as v

    dev = torch.device("cuda", 0)
    out_dim = in_dim = 4096
    r, alpha, batch = 16, 32.0, 8192
    ctx_new, ctx_ref = v.GpuContext(0), v.GpuContext(0)
    layer_new, w, a, b = _layer(v, ctx_new, out_dim, in_dim, r, alpha, 43)
    layer_ref, _, _, _ = _layer(v, ctx_ref, out_dim, in_dim, r, alpha, 43)
    gen = torch.Generator(device=dev).manual_seed(9)
    x = torch.randn(batch, in_dim, generator=gen, device=dev).to(torch.bfloat16)
    y_new = torch.zeros(batch, out_dim, device=dev, dtype=torch.bfloat16)
    y_ref = torch.zeros(batch, out_dim, device=dev, dtype=torch.bfloat16)
    small = torch.zeros(64, in_dim, device=dev, dtype=torch.bfloat16)
    # first call on the device: resolves the scratch array's address (start-up work, allowed to touch the driver)
    layer_new.forward_dev_noalloc(small.data_ptr(), 64, y_new.data_ptr())
    ctx_new.synchronize()
    torch.cuda.synchronize()
    free0, _ = torch.cuda.mem_get_info(dev)
    for _ in range(2):
        layer_new.forward_dev_noalloc(x.data_ptr(), batch, y_new.data_ptr())
    ctx_new.synchronize()
    free1, _ = torch.cuda.mem_get_info(dev)
    assert free1 == free0, (free0, free1)
    layer_ref.forward_dev(x.data_ptr(), batch, y_ref.data_ptr(), v.DTYPE_BF16)
    ctx_ref.synchronize()
    free2, _ = torch.cuda.mem_get_info(dev)
    assert free2 < free1, "the regular entry point was expected to grow its scratch arena"
    new, ref = y_new.float().cpu().numpy(), y_ref.float().cpu().numpy()
    assert rel_fro(new, ref) <= 5e-3
    # sampled rows against the CPU oracle (rows are independent)
    rows = np.array([0, 1, 127, 128, 4095, 4096, 8190, 8191])
    wd = oracle.quantize_nf4(w, out_dim, in_dim).dequantize()
    xs = x[torch.from_numpy(rows).to(dev)].float().cpu().numpy().reshape(-1)
    want = oracle.qlora_forward(xs, rows.size, wd, out_dim, in_dim, a, b, r, alpha)
    assert rel_fro(new.reshape(batch, out_dim)[rows], want) <= 5e-3
