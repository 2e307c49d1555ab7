"""The CUDA quantiser replaces the reference's 16-way nearest-level scan (quant.rs:263-278) by 15
decision thresholds on the divided target.  This test re-derives the thresholds from the oracle's scan by
bisection over fp32 bit patterns, checks that they are exactly the constants compiled into the kernel,
and checks the counting rule against the scan on dense neighbourhoods, random targets and specials."""
import os
import re

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _key(f):
    u = int(np.float32(f).view(np.uint32))
    return (u ^ 0xFFFFFFFF) if u & 0x80000000 else (u | 0x80000000)


def _unkey(k):
    u = (k & 0x7FFFFFFF) if k & 0x80000000 else (k ^ 0xFFFFFFFF)
    return np.uint32(u).view(np.float32)


def _kernel_thresholds():
    src = open(os.path.join(ROOT, "vkqlora", "rs_b200", "csrc", "quant_kernels.cu")).read()
    body = re.search(r"kT\[15\]\s*=\s*\{([^}]*)\}", src).group(1)
    return [int(x, 16) for x in re.findall(r"0x[0-9a-fA-F]+", body)]


def test_thresholds_match_the_scan(oracle):
    lv = oracle.nf4_levels()
    derived = []
    for i in range(15):
        lo, hi = _key(lv[i]), _key(lv[i + 1])
        assert oracle.nf4_code_of_target(_unkey(lo)) == i and oracle.nf4_code_of_target(_unkey(hi)) == i + 1
        while hi - lo > 1:
            mid = (lo + hi) // 2
            if oracle.nf4_code_of_target(_unkey(mid)) >= i + 1:
                hi = mid
            else:
                lo = mid
        derived.append(int(_unkey(hi).view(np.uint32)))
    assert derived == _kernel_thresholds()

    thr = np.array(derived, np.uint32).view(np.float32)

    def by_count(t):
        return 0 if t != t else int(np.sum(np.float32(t) >= thr))

    rng = np.random.default_rng(0)
    # Reachable targets are w/absmax with |w| <= absmax, i.e. |t| <= 1, or NaN (inf/inf, NaN input).
    # +-inf cannot occur (the scan would answer 0 there, the counting rule 15 / 0).
    cases = [np.float32(v) for v in (0.0, -0.0, 1.0, -1.0, np.nan, 1e-45, -1e-45)]
    for t in thr:  # +-300 ulps around every threshold
        k = _key(t)
        cases += [_unkey(k + d) for d in range(-300, 301)]
    for l in lv:
        k = _key(l)
        cases += [_unkey(k + d) for d in range(-50, 51)]
    cases += list(rng.uniform(-1.0, 1.0, 20000).astype(np.float32))
    for t in cases:
        assert by_count(t) == oracle.nf4_code_of_target(t), float(t)


def test_fast_path_bin_table(oracle):
    """The quantise kernel first classifies an approximate target by a 32-bin table: bin b names the one
    threshold k_b that targets of the bin can reach, and the code is k_b + (t >= T[k_b]).  Check, with the
    kernel's own constants, that this equals the scan for every target whose distance to T[k_b] is at
    least the kernel's 1e-6 guard band (closer ones are redone exactly by the kernel)."""
    src = open(os.path.join(ROOT, "vkqlora", "rs_b200", "csrc", "quant_kernels.cu")).read()
    scale = np.float32(re.search(r"kBinScale\s*=\s*([0-9.]+)f", src).group(1))
    m = re.search(r"\(lane & 16\) \? (0x[0-9A-Fa-f]+)ull : (0x[0-9A-Fa-f]+)ull", src)
    hi, lo = int(m.group(1), 16), int(m.group(2), 16)
    ks = [(lo >> (4 * i)) & 15 for i in range(16)] + [(hi >> (4 * i)) & 15 for i in range(16)]
    thr = np.array(_kernel_thresholds(), np.uint32).view(np.float32)

    def bin_of(t):  # int(fma(t, scale, 16)) with a single rounding, as __fmaf_rn + __float2int_rz
        return int(np.float32(np.float64(t) * np.float64(scale) + 16.0))

    # every threshold other than k_b is far outside bin b (so an approximate target cannot cross it)
    for b in range(32):
        lo_t, hi_t = (b - 16) / float(scale), (b + 1 - 16) / float(scale)
        for i in range(15):
            if i != ks[b]:
                assert thr[i] < lo_t - 1e-3 or thr[i] > hi_t + 1e-3, (b, i)
    rng = np.random.default_rng(1)
    cases = list(rng.uniform(-1.0, 1.0, 20000).astype(np.float32)) + [np.float32(x) for x in (-1.0, 1.0, 0.0, -0.0)]
    cases += [np.float32((b - 16) / float(scale) + d) for b in range(1, 32) for d in (-1e-6, -1e-7, 0.0, 1e-7, 1e-6)]
    for t in thr:
        k = _key(t)
        cases += [_unkey(k + d) for d in (-400, -100, -20, 20, 100, 400)]
    checked = 0
    for t in cases:
        if abs(float(t)) > 1.0:
            continue
        b = bin_of(t)
        assert 0 <= b <= 31, float(t)
        k = ks[b]
        if abs(np.float32(t - thr[k])) < 1e-6:
            continue  # inside the guard band: the kernel takes the exact path
        assert k + int(t >= thr[k]) == oracle.nf4_code_of_target(t), float(t)
        checked += 1
    assert checked > 20000
