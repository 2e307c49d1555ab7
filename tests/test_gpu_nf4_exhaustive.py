"""Exhaustive GPU parity of the NF4 code selection and the scale decode.

The quantise kernels do not run the reference's 16-way nearest-level scan (qlora-core/src/quant.rs:263-278):
they count decision thresholds on the divided target, and the block-64 kernel first classifies an
approximate quotient and redoes a guard band exactly.  Random data reach the places where those shortcuts
could differ from the scan only by chance, so this file sweeps them on purpose:

  * every fp32 target in [-1, 1] (2.13e9 bit patterns) through the kernels' threshold routine, compared with
    the CPU oracle's scan of the same bit patterns;
  * every weight bit pattern with |w| <= absmax, for dozens of block absmax values that are no powers of two,
    through the kernel's fast path, compared on the device with the code of the IEEE quotient w / absmax;
  * 16 384 blocks with random absmax whose elements sit on, and 1-2 ulp beside, the product
    threshold * absmax, through the real quantise kernel, compared with the oracle's quantise;
  * all 256 absmax codes under 64 second-level absmax values through block_scales / dequantize
    (quant.rs:212-221, 157-167).
All comparisons are bit-exact.
"""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

ONE = 0x3F800000      # bits of 1.0f
NEG = 0x80000000


@pytest.fixture(scope="module")
def v():
    import vkqlora.rs_b200 as v

    return v


def _gpu_codes(v, ctx, first_bits, count):
    from vkqlora.rs_b200 import _lib

    out = np.empty((count + 1) // 2, np.uint8)
    _lib.check(_lib.lib.qlc_selftest_nf4_codes_of_targets(ctx._h, first_bits, count, out.ctypes.data, out.size))
    return out


def test_threshold_routine_equals_the_scan_for_every_target_in_the_unit_interval(v, oracle):
    ctx = v.GpuContext(0)
    chunk = 1 << 26
    checked = 0
    for sign in (0, NEG):
        first, end = sign, sign + ONE + 1  # 0.0 .. 1.0 (or -0.0 .. -1.0) inclusive
        while first < end:
            n = min(chunk, end - first)
            got = _gpu_codes(v, ctx, first, n)
            want = oracle.nf4_codes_of_target_bits(first, n)
            if not np.array_equal(got, want):
                bad = int(np.flatnonzero(got != want)[0])
                raise AssertionError(f"codes differ near bit pattern {first + 2 * bad:#010x}: gpu {got[bad]:#04x} scan {want[bad]:#04x}")
            checked += n
            first += n
    assert checked == 2 * (ONE + 1)
    # just outside the interval (a quotient can never land there, the routine must still agree), and NaNs
    for first, n in ((ONE, 1 << 20), (NEG + ONE, 1 << 20), (0x7FC00000, 64), (0xFFC00000, 64), (0x7F800001, 64)):
        assert np.array_equal(_gpu_codes(v, ctx, first, n), oracle.nf4_codes_of_target_bits(first, n)), hex(first)


def _absmax_values():
    rng = np.random.default_rng(7)
    vals = [1.0, 0.7, 0.0123, 3.14159, 1.9999999, 1.0000001, 0.02 * 4.2, 1e-3, 37.5, 5e-7, 6.1e4,
            2e-30, 0.9e-30, 2.5e29, 1.5e30]  # the last four straddle the kernel's "normal absmax" window
    vals += list(np.exp(rng.uniform(np.log(1e-6), np.log(1e3), 25)))
    return [np.float32(x) for x in vals]


def test_fast_path_equals_the_ieee_quotient_for_every_weight_bit_pattern(v):
    from vkqlora.rs_b200 import _lib

    ctx = v.GpuContext(0)
    total_redone = 0
    for am in _absmax_values():
        top = int(np.float32(am).view(np.uint32))  # weights of the block: all bit patterns with |w| <= absmax
        for sign in (0, NEG):
            bad, redone, first_bad = C.c_uint64(), C.c_uint64(), C.c_uint32()
            _lib.check(_lib.lib.qlc_selftest_nf4_fast_path(ctx._h, C.c_float(float(am)), sign, top + 1, C.byref(bad),
                                                           C.byref(redone), C.byref(first_bad)))
            assert bad.value == 0, (float(am), hex(first_bad.value), bad.value)
            if 1e-29 < float(am) < 1e29:
                assert redone.value > 0  # the guard band was exercised
            total_redone += redone.value
    assert total_redone > 1000


def _thresholds(oracle):
    """The 15 decision thresholds of the scan, by bisection over bit patterns (as tests/test_nf4_thresholds.py)."""
    lv = oracle.nf4_levels()

    def key(f):
        u = int(np.float32(f).view(np.uint32))
        return (u ^ 0xFFFFFFFF) if u & NEG else (u | NEG)

    def unkey(k):
        return np.uint32((k & 0x7FFFFFFF) if k & NEG else (k ^ 0xFFFFFFFF)).view(np.float32)

    out = []
    for i in range(15):
        lo, hi = key(lv[i]), key(lv[i + 1])
        while hi - lo > 1:
            mid = (lo + hi) // 2
            if oracle.nf4_code_of_target(unkey(mid)) >= i + 1:
                hi = mid
            else:
                lo = mid
        out.append(unkey(hi))
    return np.array(out, np.float32)


@pytest.mark.parametrize("dq", [True, False])
def test_quantize_kernel_on_threshold_neighbourhoods_with_random_absmax(v, oracle, dq):
    thr = _thresholds(oracle)
    rng = np.random.default_rng(11)
    nblk = 16384
    absmax = np.exp(rng.uniform(np.log(1e-4), np.log(50.0), nblk)).astype(np.float32)  # no powers of two
    w = np.empty((nblk, 64), np.float32)
    pick = rng.integers(0, 15, (nblk, 64))
    off = rng.integers(-2, 3, (nblk, 64))
    prod = (thr[pick] * absmax[:, None]).astype(np.float32)              # fl(T_i * absmax)
    bits = prod.view(np.int32) + np.where(prod >= 0, off, -off).astype(np.int32)  # +- k ulp in value order
    w[:] = bits.view(np.float32)
    w[:, 0] = absmax * np.where(rng.integers(0, 2, nblk) == 1, 1.0, -1.0).astype(np.float32)  # pins the block absmax
    assert np.all(np.abs(w) <= absmax[:, None])
    w = w.reshape(-1)
    q = v.QuantizedTensor.quantize(w, nblk, 64, v.QuantConfig(64, dq))
    o = oracle.quantize_nf4(w, nblk, 64, 64, dq)
    assert np.array_equal(q.codes(), o.codes)
    if dq:
        assert np.array_equal(q.absmax_codes(), o.absmax_codes)
        assert np.array_equal(q.absmax2().view(np.uint32), o.absmax2.view(np.uint32))
    assert np.array_equal(q.dequantize().view(np.uint32), o.dequantize().view(np.uint32))
    # the generic (any block size) kernels take the IEEE quotient directly: same data, blocks of 32
    q32 = v.QuantizedTensor.quantize(w, nblk, 64, v.QuantConfig(32, dq))
    assert np.array_equal(q32.codes(), oracle.quantize_nf4(w, nblk, 64, 32, dq).codes)


def test_scale_decode_of_all_256_codes(v, oracle):
    rng = np.random.default_rng(5)
    a2 = [0.0, 1.0, 127.0, 1e-38, 3e-39, 1e-45, 3.4e38, 0.02, 0.0834, 1.0 / 127.0, np.inf]
    a2 += list(np.exp(rng.uniform(np.log(1e-30), np.log(1e30), 64 - len(a2))))
    a2 = np.array(a2, np.float32)
    nb = 256 * a2.size
    absmax_codes = np.tile(np.arange(256, dtype=np.uint8), a2.size)  # every i8 code, -128 included
    codes = rng.integers(0, 256, nb * 32).astype(np.uint8)            # random nibbles: all 16 levels everywhere
    q = v.QuantizedTensor.from_double_quant_parts(nb, 64, 64, codes, absmax_codes, a2)
    assert q.uses_double_quant() and q.num_blocks() == nb
    assert np.array_equal(q.codes(), codes) and np.array_equal(q.absmax_codes(), absmax_codes)
    want_scales = oracle.block_scales_dq(absmax_codes, a2)
    got_scales = q.block_scales()
    nan = np.isnan(want_scales)  # 0 * inf
    assert np.array_equal(nan, np.isnan(got_scales))
    assert np.array_equal(got_scales.view(np.uint32)[~nan], want_scales.view(np.uint32)[~nan])
    want = oracle.dequantize(codes, want_scales, nb * 64, 64)
    got = q.dequantize()
    nan = np.isnan(want)
    assert np.array_equal(nan, np.isnan(got))
    assert np.array_equal(got.view(np.uint32)[~nan], want.view(np.uint32)[~nan])
    # the same payload through the bf16 streaming kernel: round-to-nearest-even of the fp32 value
    import torch
    from refdata import to_bf16_bits

    out = torch.empty(nb * 64, dtype=torch.bfloat16, device="cuda")
    q.dequantize_dev(out.data_ptr(), v.DTYPE_BF16)
    q._ctx.synchronize()
    got_b = out.view(torch.int16).cpu().numpy().view(np.uint16)
    assert np.array_equal(got_b[~nan], to_bf16_bits(want)[~nan])
    # wrong lengths are refused like from_raw_parts (quant.rs:186-199)
    with pytest.raises(v.ShapeMismatch):
        v.QuantizedTensor.from_double_quant_parts(nb, 64, 64, codes, absmax_codes[:-1], a2)
    with pytest.raises(v.ShapeMismatch):
        v.QuantizedTensor.from_double_quant_parts(nb, 64, 64, codes, absmax_codes, a2[:-1])
