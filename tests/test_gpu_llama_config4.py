"""Model-level parity at the dimensions of benchmark configuration 4 (SmolLM-135M shape: hidden 576, 9 query heads on 3
key/value heads, MLP 1536, vocabulary 49 152) and in the reference's own projection modes.

  * one and two decoder layers at the full width, 2 sequences of 192 tokens (three 64-position attention tiles,
    sequences sharing a tile on the tensor-core path), all seven projections NF4, adapters on q and v:
    exact fp32 mode within 2e-5 (logits) / 2e-4 (adapter gradients) of the numpy restatement of
    qlora-model/src/llama.rs:310-326, 385-412; bf16 tensor-core mode within the bounds written below, each no
    looser than twice the error measured on a B200.
  * the reference's standard configurations: AdapterConfig::qv (only q and v quantised, the other five
    projections frozen fp32, llama.rs:87-93, 228-249) and AdapterConfig::none (every projection raw, forward only,
    qlora-model/tests/parity.rs:21).  The oracle multiplies by the ORIGINAL fp32 weights for the raw kinds.
"""
import numpy as np
import pytest

from oracle import np_llama as nl
from refdata import rel_fro

pytestmark = pytest.mark.gpu

SMOLLM_WIDTH = dict(hidden=576, heads=9, kv_heads=3, intermediate=1536, vocab=49152)


@pytest.fixture(scope="module")
def v():
    import vkqlora.rs_b200 as v

    return v


def _build(v, ctx, cfg_kw, seed, rank, alpha, targets, quantize, scale):
    """quantize: the kinds that are NF4-quantised on the GPU (None = all seven).  The oracle gets the dequantised
    weights for those and keeps the original fp32 matrices for the raw ones."""
    from vkqlora.rs_b200 import llama

    ocfg = nl.LlamaConfig(**cfg_kw)
    ref = nl.random_model(ocfg, seed=seed, targets=targets, rank=rank, alpha=alpha, scale=scale)
    m = llama.LlamaModel(llama.LlamaConfig(**cfg_kw), ref.embed, ref.final_norm, ctx)
    quantised = nl.KINDS if quantize is None else tuple(quantize)
    for li, L in enumerate(ref.layers):
        m.set_layer(li, L.attn_norm, L.mlp_norm, {k: L.proj[k].w for k in nl.KINDS}, quantize=quantize)
        for k in targets:
            m.attach_adapter(li, k, L.proj[k].a, L.proj[k].b, rank, alpha)
        for k in set(quantised) | set(targets):  # an adapter target is always quantised
            L.proj[k].w = m.dequantized_weight(li, k)
    return m, ref, ocfg


def _oracle(ref, ids, n_seq, seq_len, dlogits=None):
    logits = np.concatenate([ref.forward(ids[s * seq_len:(s + 1) * seq_len]) for s in range(n_seq)])
    grads = {}
    if dlogits is not None:
        for s in range(n_seq):
            g = ref.backward(ids[s * seq_len:(s + 1) * seq_len], dlogits[s * seq_len:(s + 1) * seq_len])
            for key, (ga, gb) in g.items():
                grads[key] = (grads[key][0] + ga, grads[key][1] + gb) if key in grads else (ga, gb)
    return logits, grads


def _inputs(cfg, n_seq, seq_len, seed):
    rng = np.random.default_rng(seed)
    ids = rng.integers(0, cfg.vocab, n_seq * seq_len)
    dlogits = (rng.standard_normal((n_seq * seq_len, cfg.vocab)) * 0.01).astype(np.float32)
    return ids, dlogits


@pytest.mark.parametrize("layers", [1, 2])
def test_config4_width_exact_and_bf16(v, layers):
    n_seq, seq_len, rank, alpha = 2, 192, 8, 16.0
    kw = dict(SMOLLM_WIDTH, layers=layers)
    ctx = v.GpuContext(0)
    ctx.set_precision(v.PRECISION_FP32_EXACT)
    m, ref, cfg = _build(v, ctx, kw, seed=61 + layers, rank=rank, alpha=alpha, targets=("q", "v"), quantize=None, scale=0.04)
    ids, dlogits = _inputs(cfg, n_seq, seq_len, 20 + layers)
    want_logits, want_grads = _oracle(ref, ids, n_seq, seq_len, dlogits)
    assert set(want_grads) == {(l, k) for l in range(layers) for k in ("q", "v")}

    # exact fp32 mode: only summation order differs from the oracle
    e = rel_fro(m.forward(ids, n_seq, seq_len), want_logits)
    assert e <= 2e-5, e
    m.backward(ids, dlogits, n_seq, seq_len)
    for (li, kind), (ga, gb) in want_grads.items():
        a, b = m.adapter_grads(li, kind, rank)
        assert rel_fro(a, ga) <= 2e-4 and rel_fro(b, gb) <= 2e-4, (li, kind, rel_fro(a, ga), rel_fro(b, gb))

    # bf16 tensor-core mode (bf16 activation pipeline, tcgen05 attention, bf16 LM head).
    # Measured on a B200 at these dimensions: see BF16_BOUNDS; every bound is <= 2x the measured error.
    ctx.set_precision(v.PRECISION_BF16)
    e = rel_fro(m.forward(ids, n_seq, seq_len), want_logits)
    worst = {"logits": e, "grad_a": 0.0, "grad_b": 0.0}
    m.backward(ids, dlogits, n_seq, seq_len)
    for (li, kind), (ga, gb) in want_grads.items():
        a, b = m.adapter_grads(li, kind, rank)
        worst["grad_a"] = max(worst["grad_a"], rel_fro(a, ga))
        worst["grad_b"] = max(worst["grad_b"], rel_fro(b, gb))
    print(f"config-4 width, {layers} layer(s), bf16 mode, measured:", {k: f"{x:.2e}" for k, x in worst.items()})
    for k, bound in BF16_BOUNDS[layers].items():
        assert worst[k] <= bound, (k, worst[k], bound)


# Relative Frobenius error of the bf16 mode against the fp32 oracle, by number of layers.  Measured on a B200:
# 1 layer: logits 4.49e-3, grad_a 8.70e-3, grad_b 8.97e-3; 2 layers: logits 6.05e-3, grad_a 1.22e-2, grad_b 1.22e-2.
BF16_BOUNDS = {1: {"logits": 8.9e-3, "grad_a": 1.7e-2, "grad_b": 1.79e-2},
               2: {"logits": 1.2e-2, "grad_a": 2.4e-2, "grad_b": 2.4e-2}}


def test_reference_qv_configuration_other_projections_raw(v):
    """AdapterConfig::qv: q and v are NF4 + adapter, k / o / gate / up / down stay frozen fp32.  In exact mode the
    raw projections multiply by the original fp32 weights, so the model carries NF4 error only where the
    reference's does."""
    kw = dict(hidden=128, layers=2, heads=2, kv_heads=1, intermediate=192, vocab=96)
    n_seq, seq_len, rank, alpha = 2, 70, 4, 8.0
    ctx = v.GpuContext(0)
    ctx.set_precision(v.PRECISION_FP32_EXACT)
    m, ref, cfg = _build(v, ctx, kw, seed=71, rank=rank, alpha=alpha, targets=("q", "v"), quantize=("q", "v"), scale=0.08)
    # the raw kinds were NOT replaced by a quantised round trip
    from vkqlora.rs_b200 import _lib

    for k in ("k", "o", "gate", "up", "down"):
        layer = _lib.lib.qlc_llama_projection(m._h, 0, nl.KINDS.index(k))
        assert not _lib.lib.qlc_layer_weight(layer), k
    ids, dlogits = _inputs(cfg, n_seq, seq_len, 31)
    dlogits *= 10
    want_logits, want_grads = _oracle(ref, ids, n_seq, seq_len, dlogits)
    assert rel_fro(m.forward(ids, n_seq, seq_len), want_logits) <= 2e-5
    m.backward(ids, dlogits, n_seq, seq_len)
    for (li, kind), (ga, gb) in want_grads.items():
        a, b = m.adapter_grads(li, kind, rank)
        assert rel_fro(a, ga) <= 2e-4 and rel_fro(b, gb) <= 2e-4, (li, kind, rel_fro(a, ga), rel_fro(b, gb))
    # the same model on the tensor-core path: raw weights rounded to bf16, both operands by TMA
    ctx.set_precision(v.PRECISION_BF16)
    assert rel_fro(m.forward(ids, n_seq, seq_len), want_logits) <= 2e-2
    m.backward(ids, dlogits, n_seq, seq_len)
    for (li, kind), (ga, gb) in want_grads.items():
        a, b = m.adapter_grads(li, kind, rank)
        assert rel_fro(a, ga) <= 5e-2 and rel_fro(b, gb) <= 5e-2, (li, kind, rel_fro(a, ga), rel_fro(b, gb))
    # TF32 mode: quantised projections on the tensor cores in tf32, raw ones in exact fp32
    ctx.set_precision(v.PRECISION_TF32)
    assert rel_fro(m.forward(ids, n_seq, seq_len), want_logits) <= 1e-2


def test_reference_no_adapter_configuration_forward(v):
    """AdapterConfig::none (qlora-model/tests/parity.rs:21): nothing is quantised, the forward pass is a plain
    fp32 Llama; exact mode reproduces the oracle on the original weights to summation order."""
    kw = dict(hidden=128, layers=2, heads=2, kv_heads=1, intermediate=192, vocab=96)
    n_seq, seq_len = 3, 50
    ctx = v.GpuContext(0)
    ctx.set_precision(v.PRECISION_FP32_EXACT)
    m, ref, cfg = _build(v, ctx, kw, seed=73, rank=1, alpha=1.0, targets=(), quantize=(), scale=0.08)
    ids, _ = _inputs(cfg, n_seq, seq_len, 33)
    want_logits, _ = _oracle(ref, ids, n_seq, seq_len)
    assert rel_fro(m.forward(ids, n_seq, seq_len), want_logits) <= 2e-5
    ctx.set_precision(v.PRECISION_BF16)
    assert rel_fro(m.forward(ids, n_seq, seq_len), want_logits) <= 2e-2
    # attaching an adapter to a raw projection quantises it (block 64 + double quantisation) first
    o, i = cfg.proj_dims("q")
    m.attach_adapter(0, "q", np.zeros((2, i), np.float32), np.zeros((o, 2), np.float32), 2, 4.0)
    wq = m.dequantized_weight(0, "q")
    assert wq.shape == (o, i) and 0 < rel_fro(wq, ref.layers[0].proj["q"].w) < 0.2
