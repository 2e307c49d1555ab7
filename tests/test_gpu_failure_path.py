"""The path from a bounded wait that gives up to an error on the host, exercised without faulting the GPU.

Every mbarrier wait of the tensor-core kernels is bounded: on expiry the kernel stores a status word, unwinds
and returns; later tensor-core launches on the context see the raised status at their top and return at once;
qlc_ctx_synchronize reports QLC_ERR_GPU with the site and clears the status.  A healthy run never takes that
path, so a dedicated kernel takes it on purpose: one CTA, no TMA, no tensor memory, whose thread 0 waits with
the same routine (a ~1 ms limit) on a barrier nobody arrives on.  Nothing traps and nothing spins without
bound; the context keeps working."""
import time

import numpy as np
import pytest

from refdata import normal, rel_fro, to_bf16_f32

pytestmark = pytest.mark.gpu


def test_wait_timeout_becomes_gpu_error_and_the_context_recovers(oracle):
    import torch

    import vkqlora.rs_b200 as v
    from vkqlora.rs_b200 import _lib

    dev = torch.device("cuda", 0)
    ctx = v.GpuContext(0)
    ctx.set_precision(v.PRECISION_BF16)
    out_dim, in_dim, r, batch = 256, 192, 8, 300
    w = normal(1, out_dim * in_dim, 0.02)
    a, b = normal(2, r * in_dim, 0.07), normal(3, out_dim * r, 0.01)
    layer = v.QloraLinear.new(w, out_dim, in_dim, v.QuantConfig(), v.LoraAdapter(a, b, in_dim, out_dim, r, 16.0), ctx)
    xh = to_bf16_f32(normal(4, batch * in_dim, 1.0))
    x = torch.from_numpy(xh).to(dev).to(torch.bfloat16).reshape(batch, in_dim)
    y = torch.full((batch, out_dim), 7.0, device=dev, dtype=torch.bfloat16)
    torch.cuda.synchronize()
    ctx.synchronize()

    # 1. the wait gives up after ~2e6 cycles (about a millisecond) and the kernel returns by itself
    t0 = time.perf_counter()
    _lib.check(_lib.lib.qlc_selftest_wait_timeout(ctx._h, 2_000_000))
    # 2. a forward pass queued behind it must not run: its kernels return at their top
    layer.forward_dev(x.data_ptr(), batch, y.data_ptr(), v.DTYPE_BF16)
    with pytest.raises(v.GpuError) as e:
        ctx.synchronize()
    assert time.perf_counter() - t0 < 5.0
    msg = str(e.value)
    assert "gpu error" in msg and "status 1" in msg and "site 99" in msg and "block 0" in msg, msg
    torch.cuda.synchronize()
    assert torch.all(y == 7.0).item(), "a kernel queued after the failure wrote its output"

    # 3. the report cleared the status: the next synchronise is clean and the same call now computes
    ctx.synchronize()
    layer.forward_dev(x.data_ptr(), batch, y.data_ptr(), v.DTYPE_BF16)
    ctx.synchronize()
    q = oracle.quantize_nf4(w, out_dim, in_dim)
    want = oracle.qlora_forward(xh, batch, q.dequantize(), out_dim, in_dim, a, b, r, 16.0)
    assert rel_fro(y.float().cpu().numpy(), want) <= 5e-3

    # 4. limits outside the test range are refused on the host
    with pytest.raises(v.InvalidConfig):
        _lib.check(_lib.lib.qlc_selftest_wait_timeout(ctx._h, 0))
    with pytest.raises(v.InvalidConfig):
        _lib.check(_lib.lib.qlc_selftest_wait_timeout(ctx._h, 10**12))
