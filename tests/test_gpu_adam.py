"""GPU parity of the paged 8-bit Adam step through the C ABI vs the CPU oracle, plus the
reference's own optimiser tests (qlora-core/tests/optim.rs) replayed on the GPU."""
import numpy as np
import pytest

from refdata import normal, pattern

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def v():
    import vkqlora.rs_b200 as v

    return v


def _compare_state(opt, oopt, i):
    st, os_ = opt.get_state(i), oopt.states[i]
    assert st["step"] == os_["step"].value and st["numel"] == os_["numel"]
    # north star: 8-bit codes equal except at rounding ties; we require (and get) exact equality
    assert np.array_equal(st["m_codes"], os_["m_codes"]), "m codes"
    assert np.array_equal(st["v_codes"], os_["v_codes"]), "v codes"
    assert np.array_equal(st["m_scales"].view(np.uint32), os_["m_scales"].view(np.uint32))
    assert np.array_equal(st["v_scales"].view(np.uint32), os_["v_scales"].view(np.uint32))


@pytest.mark.parametrize("sizes,bs", [([1024], 256), ([1000, 77, 256, 4096 + 13], 256), ([300, 64], 32), ([50], 7)])
def test_adam_bitwise_vs_oracle(v, oracle, sizes, bs):
    opt = v.Adam8bit(v.AdamConfig(block_size=bs))
    oopt = oracle.Adam8bit(block_size=bs)
    p1 = [normal(10 + i, n, 0.01) for i, n in enumerate(sizes)]
    p2 = [p.copy() for p in p1]
    for t in range(6):
        g = [normal(100 * t + i, n, 0.01) for i, n in enumerate(sizes)]
        s1 = opt.step(p1, g)
        s2 = oopt.step(p2, g)
        assert (s1.pages_streamed, s1.state_bytes) == s2
        for i in range(len(sizes)):
            # north star asks for <= 1e-5 relative error on parameters; the kernel is bit-exact
            assert np.array_equal(p1[i].view(np.uint32), p2[i].view(np.uint32)), (t, i)
            _compare_state(opt, oopt, i)


def test_adam_bitwise_large_random(v, oracle):
    """One million elements over several steps, including zero gradients, tiny and large magnitudes:
    the kernel's prepared-reciprocal divisions must stay bit-identical to IEEE division."""
    n = 1 << 20
    rng = np.random.default_rng(3)
    p1 = [normal(50, n, 0.01)]
    p2 = [p1[0].copy()]
    opt, oopt = v.Adam8bit(), oracle.Adam8bit()
    for t in range(5):
        g = normal(200 + t, n, 0.01)
        g[rng.integers(0, n, n // 10)] = 0.0                      # sparse zeros
        g[:4096] *= np.float32(10.0) ** rng.integers(-12, 6, 4096).astype(np.float32)  # wide dynamic range
        opt.step(p1, [g])
        oopt.step(p2, [g])
        assert np.array_equal(p1[0].view(np.uint32), p2[0].view(np.uint32)), t
    _compare_state(opt, oopt, 0)


def test_fast_math_mode_stays_within_tolerance(v, oracle):
    """Opt-in relaxed arithmetic: after one step from identical state the parameters agree with the oracle to
    1e-5 relative (north-star tolerance) and the 8-bit codes differ only next to rounding boundaries; over
    several steps the trajectories stay close."""
    n = 1 << 18
    p1, p2 = [normal(60, n, 0.01)], [normal(60, n, 0.01)]
    opt, oopt = v.Adam8bit(), oracle.Adam8bit()
    opt.set_fast_math(True)
    g = normal(300, n, 0.01)
    opt.step(p1, [g])
    oopt.step(p2, [g])
    # relative to the size of the parameters (an element-wise ratio is meaningless where p - update cancels)
    diff = np.abs(p1[0].astype(np.float64) - p2[0])
    assert np.linalg.norm(diff) / np.linalg.norm(p2[0].astype(np.float64)) <= 1e-5
    assert diff.max() <= 1e-5 * np.abs(p2[0]).max(), float(diff.max())
    st, os_ = opt.get_state(0), oopt.states[0]
    for key in ("m_codes", "v_codes"):
        d = np.abs(st[key].view(np.int8).astype(np.int32) - os_[key].view(np.int8).astype(np.int32))
        assert d.max() <= 1 and np.mean(d != 0) < 1e-3, (key, int(d.max()), float(np.mean(d != 0)))
    assert np.allclose(st["m_scales"], os_["m_scales"], rtol=1e-6) and np.allclose(st["v_scales"], os_["v_scales"], rtol=1e-6)
    for t in range(4):
        g = normal(301 + t, n, 0.01)
        opt.step(p1, [g])
        oopt.step(p2, [g])
    err = np.linalg.norm(p1[0].astype(np.float64) - p2[0]) / np.linalg.norm(p2[0].astype(np.float64))
    assert err < 1e-4, err


def test_ref_tracks_fp64_reference(v):  # tests/optim.rs:27-60
    n = 64
    g = pattern(n, 13, 17, 17.0, 0.5)
    params = [np.ones(n, np.float32)]
    opt = v.Adam8bit(v.AdamConfig(lr=0.01, block_size=32))
    pr, gr, m, vv = np.ones(n), g.astype(np.float64), np.zeros(n), np.zeros(n)
    for t in range(1, 6):
        opt.step(params, [g])
        m = 0.9 * m + 0.1 * gr
        vv = 0.999 * vv + (1 - 0.999) * gr * gr
        pr = pr - 0.01 * (m / (1 - 0.9 ** t)) / (np.sqrt(vv / (1 - 0.999 ** t)) + 1e-8)
        assert np.max(np.abs(params[0] - pr)) < 5e-3


def test_ref_paging_matches_fully_resident_bitwise(v):  # tests/optim.rs:62-87
    g = pattern(256, 7, 43, 43.0, 0.5)
    pa = [np.full(256, 0.5, np.float32), np.full(256, -1.0, np.float32)]
    pb = [p.copy() for p in pa]
    oa = v.Adam8bit(v.AdamConfig(lr=0.01, block_size=16, max_resident_pages=1))
    ob = v.Adam8bit(v.AdamConfig(lr=0.01, block_size=16))
    for _ in range(3):
        sa, sb = oa.step(pa, [g, g]), ob.step(pb, [g, g])
        assert sa.pages_streamed == sb.pages_streamed == 32
        assert all(np.array_equal(x, y) for x, y in zip(pa, pb))
    assert oa.paging_info()["host_bytes"] > 0 and ob.paging_info()["host_bytes"] == 0


def test_ref_converges_and_state_is_compact(v):  # tests/optim.rs:89-131
    params = [np.full(32, 2.0, np.float32)]
    opt = v.Adam8bit(v.AdamConfig(lr=0.05, block_size=32))
    for _ in range(300):
        opt.step(params, [(np.float32(2.0) * params[0]).astype(np.float32)])
    assert np.max(np.abs(params[0])) < 0.05
    opt = v.Adam8bit()
    opt.step([np.full(1024, 0.1, np.float32)], [np.full(1024, 0.01, np.float32)])
    assert opt.state_bytes() == 2048 + 2 * 4 * 4
    with pytest.raises(v.InvalidConfig):
        v.Adam8bit(v.AdamConfig(lr=-0.1))
    with pytest.raises(v.InvalidConfig):
        v.Adam8bit(v.AdamConfig(block_size=0))
    with pytest.raises(v.ShapeMismatch):
        opt.step([np.ones(4, np.float32)], [np.ones(5, np.float32)])


def test_forced_eviction_many_tensors_bitwise(v, oracle):
    """A scaled-down benchmark configuration 3: many tensors, max_resident_pages=4 so every state page is
    evicted to pinned host memory each step; results must equal the resident run and the oracle."""
    sizes = [65536 + 256 * (i % 3) for i in range(12)]
    paged = v.Adam8bit(v.AdamConfig(max_resident_pages=4))
    resident = v.Adam8bit(v.AdamConfig())
    oopt = oracle.Adam8bit()
    p1 = [normal(20 + i, n, 0.01) for i, n in enumerate(sizes)]
    p2 = [p.copy() for p in p1]
    p3 = [p.copy() for p in p1]
    for t in range(3):
        g = [normal(1000 * t + i, n, 0.01) for i, n in enumerate(sizes)]
        paged.step(p1, g)
        resident.step(p2, g)
        oopt.step(p3, g)
        for i in range(len(sizes)):
            assert np.array_equal(p1[i], p2[i]) and np.array_equal(p1[i].view(np.uint32), p3[i].view(np.uint32)), (t, i)
    info = paged.paging_info()
    assert info["h2d_bytes_last_step"] == info["d2h_bytes_last_step"] == paged.state_bytes()
    for i in (0, 5, 11):
        _compare_state(paged, oopt, i)


@pytest.mark.gpu
def test_forced_eviction_mixed_sizes_bitwise(v, oracle):
    """Paged mode over 70 tiny tensors (more than one descriptor batch of 32, sizes that are no multiple of the
    block), one tensor of three pages and a few medium ones: neighbouring page records travel in groups, a group
    ends at the descriptor-batch limit, at the slot size and where the host records are not adjacent.  Results equal
    the resident run bit for bit, for several steps."""
    sizes = [300 + 37 * i for i in range(70)] + [2 * (1 << 20) + 5000] + [70000, 333, 1 << 20, 4097]
    paged = v.Adam8bit(v.AdamConfig(max_resident_pages=2))
    resident = v.Adam8bit(v.AdamConfig())
    p1 = [normal(50 + i, n, 0.01) for i, n in enumerate(sizes)]
    p2 = [p.copy() for p in p1]
    for t in range(3):
        g = [normal(2000 * (t + 1) + i, n, 0.01) for i, n in enumerate(sizes)]
        paged.step(p1, g)
        resident.step(p2, g)
        for i in range(len(sizes)):
            assert np.array_equal(p1[i].view(np.uint32), p2[i].view(np.uint32)), (t, i, sizes[i])
    info = paged.paging_info()
    assert info["h2d_bytes_last_step"] == info["d2h_bytes_last_step"] == paged.state_bytes()


def test_state_save_restore_continues_bitwise(v, oracle):
    """Checkpointing: get_state of every tensor, restored into a fresh optimiser with set_state, then both take
    more steps - parameters and state stay bit-identical (ParamState, optim.rs:104-126).  Once resident, once
    with the state parked in pinned host memory (max_resident_pages=2)."""
    sizes = [1000, 77, 4096 + 13, 70000]
    for pages in (None, 2):
        a = v.Adam8bit(v.AdamConfig(max_resident_pages=pages))
        pa = [normal(30 + i, n, 0.01) for i, n in enumerate(sizes)]
        for t in range(3):
            a.step(pa, [normal(500 * t + i, n, 0.01) for i, n in enumerate(sizes)])
        saved = [a.get_state(i) for i in range(len(sizes))]
        assert all(s["step"] == 3 for s in saved)
        b = v.Adam8bit(v.AdamConfig(max_resident_pages=pages))
        for i, s in enumerate(saved):
            b.set_state(i, s)
        assert b.state_bytes() == a.state_bytes()
        pb = [p.copy() for p in pa]
        for t in range(3, 6):
            g = [normal(500 * t + i, n, 0.01) for i, n in enumerate(sizes)]
            a.step(pa, g)
            b.step(pb, g)
            for i in range(len(sizes)):
                assert np.array_equal(pa[i].view(np.uint32), pb[i].view(np.uint32)), (pages, t, i)
        for i in range(len(sizes)):
            sa, sb = a.get_state(i), b.get_state(i)
            assert sa["step"] == sb["step"] == 6
            for k in ("m_codes", "v_codes", "m_scales", "v_scales"):
                assert np.array_equal(sa[k], sb[k]), (pages, i, k)
        # replacing a state in place (same index) and wrong orders / sizes
        b.set_state(1, saved[1])
        assert b.get_state(1)["step"] == 3
        with pytest.raises(v.ShapeMismatch):
            v.Adam8bit().set_state(2, saved[2])  # index 2 before 0 and 1
        bad = dict(saved[0], m_codes=saved[0]["m_codes"][:-1])
        with pytest.raises(v.ShapeMismatch):
            b.set_state(0, bad)


def test_full_size_config3_bitwise(v, oracle):
    """benchmark configuration 3 at full size: 112 tensors x 262 144 fp32 (28 layers x Q/V x {A 64x4096, B 4096x64}),
    block 256, 3 steps, fully resident and with max_resident_pages=4 (every page evicted to pinned host memory
    each step), on device buffers as the benchmark runs it.  Parameters and 8-bit state of both runs equal the
    CPU oracle's bit for bit; the oracle steps a sample of the tensors (all tensors are independent)."""
    import torch

    n_t, numel = 112, 262144
    dev = torch.device("cuda", 0)
    ctx = v.GpuContext(0)
    host_p = [normal(6000 + i, numel, 0.01) for i in range(n_t)]
    runs = {}
    for name, pages in (("resident", None), ("paged", 4)):
        opt = v.Adam8bit(v.AdamConfig(max_resident_pages=pages), ctx)
        params = [torch.from_numpy(p).to(dev) for p in host_p]
        for t in range(3):
            grads = [torch.from_numpy(normal(7000 + 1000 * t + i, numel, 0.01)).to(dev) for i in range(n_t)]
            torch.cuda.synchronize()
            st = opt.step_dev([p.data_ptr() for p in params], [g.data_ptr() for g in grads], [numel] * n_t)
            ctx.synchronize()
            assert st.pages_streamed == n_t * numel // 256 and st.state_bytes == 59637760
        runs[name] = (opt, [p.cpu().numpy() for p in params])
    info = runs["paged"][0].paging_info()
    assert info["host_bytes"] == 59637760 and info["h2d_bytes_last_step"] == 59637760
    for i in range(n_t):
        assert np.array_equal(runs["resident"][1][i].view(np.uint32), runs["paged"][1][i].view(np.uint32)), i
    sample = [0, 1, 55, 110, 111]
    for i in sample:
        oopt = oracle.Adam8bit()
        p = [host_p[i].copy()]
        for t in range(3):
            oopt.step(p, [normal(7000 + 1000 * t + i, numel, 0.01)])
        for name in runs:
            assert np.array_equal(runs[name][1][i].view(np.uint32), p[0].view(np.uint32)), (name, i)
            st, os_ = runs[name][0].get_state(i), oopt.states[0]
            assert st["step"] == 3
            assert np.array_equal(st["m_codes"], os_["m_codes"]) and np.array_equal(st["v_codes"], os_["v_codes"])
            assert np.array_equal(st["m_scales"].view(np.uint32), os_["m_scales"].view(np.uint32))
            assert np.array_equal(st["v_scales"].view(np.uint32), os_["v_scales"].view(np.uint32))


def test_branch_free_sqrt_and_div_equal_the_ieee_operations(v):
    """The exact kernel's straight-line square root and division must round like IEEE sqrt and division wherever
    the kernel uses them: the square root is swept over EVERY fp32 value in [2^-101, 2^101) (the kernel's window is
    [2^-80, 2^80]), the division over 2^33 seeded operand pairs spanning its operand windows."""
    import ctypes as C

    from vkqlora.rs_b200 import _lib

    ctx = v.GpuContext(0)
    bad, first = C.c_uint64(), C.c_uint64()
    lo, hi = (127 - 101) << 23, (127 + 101) << 23
    _lib.check(_lib.lib.qlc_selftest_adam_math(ctx._h, 0, lo, hi - lo, 0, C.byref(bad), C.byref(first)))
    assert bad.value == 0, (bad.value, hex(lo + first.value))
    for seed in (1, 2):
        _lib.check(_lib.lib.qlc_selftest_adam_math(ctx._h, 1, 0, 1 << 32, seed << 40, C.byref(bad), C.byref(first)))
        assert bad.value == 0, (seed, bad.value, first.value)


def test_adam_bitwise_outside_the_fast_windows(v, oracle):
    """Gradients and state that leave the branch-free path's operand windows (tiny, huge, zero, mixed within one
    thread's eight elements) and step constants outside its windows: the kernel must fall back to the IEEE
    operations and stay bit-identical to the oracle."""
    n = 8192
    rng = np.random.default_rng(21)
    scales = np.float32(10.0) ** rng.integers(-30, 20, n).astype(np.float32)   # per-element magnitudes 1e-30 .. 1e19
    for cfg in (dict(), dict(lr=1e-12), dict(eps=2000.0), dict(beta2=0.9999999)):
        opt, oopt = v.Adam8bit(v.AdamConfig(**cfg)), oracle.Adam8bit(**cfg)
        p1 = [normal(70, n, 0.01)]
        p2 = [p1[0].copy()]
        for t in range(4):
            g = (normal(700 + t, n, 1.0) * scales).astype(np.float32)
            g[rng.integers(0, n, n // 8)] = 0.0
            if t == 2:
                g[:] = 0.0          # a whole step without gradient
            opt.step(p1, [g])
            oopt.step(p2, [g])
            assert np.array_equal(p1[0].view(np.uint32), p2[0].view(np.uint32)), (cfg, t)
        _compare_state(opt, oopt, 0)


@pytest.mark.parametrize("mode", ["slots", "hybrid"])
def test_paged_modes_match_resident_bitwise(mode, tmp_path):
    """QLC_ADAM_PAGED_MODE is read once per process, so the two copy-based forms of a paged step (pages through
    device slots both ways / on the way in only) run in a process of their own: parameters and 8-bit state after
    three steps equal the resident optimiser's bit for bit, as in the default (in-place) form the other tests use."""
    import os
    import subprocess
    import sys
    here = os.path.dirname(os.path.abspath(__file__))
    code = f"""
import sys; sys.path.insert(0, {os.path.dirname(here)!r}); sys.path.insert(0, {here!r})
import numpy as np, vkqlora.rs_b200 as v
from refdata import normal
sizes = [300000, 77, 4096 + 13, 1100000]
a = v.Adam8bit(v.AdamConfig(max_resident_pages=2)); b = v.Adam8bit(v.AdamConfig())
pa = [normal(30 + i, n, 0.01) for i, n in enumerate(sizes)]; pb = [p.copy() for p in pa]
for t in range(3):
    g = [normal(500 * t + i, n, 0.01) for i, n in enumerate(sizes)]
    a.step(pa, g); b.step(pb, g)
for i in range(len(sizes)):
    assert np.array_equal(pa[i].view(np.uint32), pb[i].view(np.uint32)), i
    sa, sb = a.get_state(i), b.get_state(i)
    for k in ("m_codes", "v_codes", "m_scales", "v_scales"):
        assert np.array_equal(sa[k], sb[k]), (i, k)
assert a.paging_info()["host_bytes"] > 0
print("ok")
"""
    env = dict(os.environ, QLC_ADAM_PAGED_MODE=mode)
    out = subprocess.run([sys.executable, "-c", code], env=env, capture_output=True, text=True, timeout=300)
    assert out.returncode == 0 and "ok" in out.stdout, out.stderr[-2000:]
