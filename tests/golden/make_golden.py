#!/usr/bin/env python
"""Generates the golden fixtures in this directory with the CPU oracle (oracle/qlora_oracle.c).

    python tests/golden/make_golden.py

The reference (Rust) cannot be executed on the build machine, so these vectors are outputs of the C
restatement, which is itself pinned by the reference's own tests (tests/test_oracle_*.py) and by an
independent numpy restatement (tests/test_oracle_cross.py).  They freeze the oracle's behaviour (any later
edit that changes a bit fails tests/test_golden.py) and are replayed on the GPU bit-for-bit.
Inputs are regenerated from seeds by the tests; only outputs are stored.
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

from oracle import c_oracle as orc  # noqa: E402
from refdata import normal, pattern  # noqa: E402

QUANT_CASES = {  # name -> (weights factory, rows, cols, block_size, double_quant)
    "normal_576x576": (lambda: normal(1, 576 * 576, 0.02), 576, 576, 64, True),
    "normal_18x20": (lambda: normal(2, 18 * 20, 0.02), 18, 20, 64, True),
    "ramp_2x5": (lambda: (np.arange(10, dtype=np.float32) / np.float32(10)).astype(np.float32), 2, 5, 64, True),
    "ramp_10x10": (lambda: ((np.arange(100, dtype=np.float32) - 50) / 50).astype(np.float32), 10, 10, 64, True),
    "pattern_16x32_plain": (lambda: pattern(512, 7, 31, 31.0, 0.5), 16, 32, 64, False),
    "normal_37x53_b32": (lambda: normal(3, 37 * 53, 0.05), 37, 53, 32, True),
}

LAYER_CASES = {  # name -> (out_dim, in_dim, r, batch, alpha)
    "c1_576": (576, 576, 8, 32, 16.0),  # benchmark configuration 1
    "odd_18x20": (18, 20, 5, 3, 8.0),   # qlora-wgpu/tests/gpu_backward.rs:60
    "tiny_3x4": (3, 4, 2, 2, 8.0),      # qlora-core/tests/qlora.rs:91
}


def layer_inputs(name):
    out_dim, in_dim, r, batch, alpha = LAYER_CASES[name]
    w = normal(1, out_dim * in_dim, 0.02)
    a = normal(2, r * in_dim, 1.0 / np.sqrt(in_dim))
    b = normal(3, out_dim * r, 0.01)
    x, dy = normal(4, batch * in_dim), normal(5, batch * out_dim)
    return w, a, b, x, dy


ADAM_SIZES, ADAM_STEPS = [1024, 1000, 77], 4


def adam_inputs():
    params = [normal(10 + i, n, 0.01) for i, n in enumerate(ADAM_SIZES)]
    grads = [[normal(100 * t + i, n, 0.01) for i, n in enumerate(ADAM_SIZES)] for t in range(ADAM_STEPS)]
    return params, grads


def main():
    out = {}
    for name, (mk, rows, cols, bs, dq) in QUANT_CASES.items():
        q = orc.quantize_nf4(mk(), rows, cols, bs, dq)
        out[f"quant/{name}/codes"] = q.codes
        out[f"quant/{name}/scales"] = q.block_scales()
        if dq:
            out[f"quant/{name}/absmax_codes"] = q.absmax_codes
            out[f"quant/{name}/absmax2"] = q.absmax2
        out[f"quant/{name}/dequant_crc"] = np.array([np.bitwise_xor.reduce(q.dequantize().view(np.uint32)),
                                                    np.sum(q.dequantize().view(np.uint32).astype(np.uint64)) & 0xFFFFFFFF],
                                                   dtype=np.uint64)
    for name, (out_dim, in_dim, r, batch, alpha) in LAYER_CASES.items():
        w, a, b, x, dy = layer_inputs(name)
        wd = orc.quantize_nf4(w, out_dim, in_dim).dequantize()
        out[f"layer/{name}/y"] = orc.qlora_forward(x, batch, wd, out_dim, in_dim, a, b, r, alpha)
        gx, ga, gb = orc.qlora_backward(x, dy, batch, wd, out_dim, in_dim, a, b, r, alpha)
        out[f"layer/{name}/grad_x"], out[f"layer/{name}/grad_a"], out[f"layer/{name}/grad_b"] = gx, ga, gb
    params, grads = adam_inputs()
    opt = orc.Adam8bit()
    for t in range(ADAM_STEPS):
        opt.step(params, grads[t])
    for i, p in enumerate(params):
        out[f"adam/{i}/param"] = p
        out[f"adam/{i}/m_codes"] = opt.states[i]["m_codes"]
        out[f"adam/{i}/v_codes"] = opt.states[i]["v_codes"]
        out[f"adam/{i}/m_scales"] = opt.states[i]["m_scales"]
        out[f"adam/{i}/v_scales"] = opt.states[i]["v_scales"]
    path = os.path.join(HERE, "oracle_golden.npz")
    np.savez_compressed(path, **out)
    print(path, os.path.getsize(path), "bytes,", len(out), "arrays")


if __name__ == "__main__":
    main()
