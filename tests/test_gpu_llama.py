"""Llama decoder around the QLoRA linears (qlc_llama_*) against the numpy restatement of
qlora-model/src/llama.rs (oracle/np_llama.py): logits, adapter gradients, loss, and a training step.
The oracle is given the DEQUANTISED weights of every projection as raw fp32 matrices - mathematically what
the reference's Proj::Qlora computes (llama.rs:106-114) - so the comparison isolates the model code."""
import numpy as np
import pytest

from oracle import np_llama as nl
from refdata import rel_fro


@pytest.fixture(scope="module")
def v():
    import vkqlora.rs_b200 as v

    return v


def _build(v, ctx, cfg_kw, seed, rank, alpha, targets=("q", "v")):
    from vkqlora.rs_b200 import llama
    ocfg = nl.LlamaConfig(**cfg_kw)
    ref = nl.random_model(ocfg, seed=seed, targets=targets, rank=rank, alpha=alpha, scale=0.08)
    cfg = llama.LlamaConfig(**cfg_kw)
    m = llama.LlamaModel(cfg, ref.embed, ref.final_norm, ctx)
    for li, L in enumerate(ref.layers):
        m.set_layer(li, L.attn_norm, L.mlp_norm, {k: L.proj[k].w for k in nl.KINDS})
        for k in targets:
            m.attach_adapter(li, k, L.proj[k].a, L.proj[k].b, rank, alpha)
        for k in nl.KINDS:                       # the oracle multiplies by what the GPU multiplies by
            L.proj[k].w = m.dequantized_weight(li, k)
    return m, ref, ocfg


def _oracle_batch(ref, ids, n_seq, seq_len, dlogits=None):
    logits = np.concatenate([ref.forward(ids[s * seq_len:(s + 1) * seq_len]) for s in range(n_seq)])
    grads = None
    if dlogits is not None:
        grads = {}
        for s in range(n_seq):
            g = ref.backward(ids[s * seq_len:(s + 1) * seq_len], dlogits[s * seq_len:(s + 1) * seq_len])
            for key, (ga, gb) in g.items():
                if key in grads:
                    grads[key] = (grads[key][0] + ga, grads[key][1] + gb)
                else:
                    grads[key] = (ga, gb)
    return logits, grads


TINY = dict(hidden=128, layers=2, heads=2, kv_heads=1, intermediate=192, vocab=96)


@pytest.mark.gpu
def test_model_forward_backward_exact_mode_matches_oracle(v):
    """fp32 everywhere (exact linears, exact LM head): only summation order differs from the oracle."""
    ctx = v.GpuContext(0)
    ctx.set_precision(v.PRECISION_FP32_EXACT)
    rank, alpha, n_seq, seq_len = 4, 8.0, 2, 24      # 24 positions: a ragged 64-row attention tile
    m, ref, cfg = _build(v, ctx, TINY, seed=5, rank=rank, alpha=alpha)
    rng = np.random.default_rng(0)
    ids = rng.integers(0, cfg.vocab, n_seq * seq_len)
    dlogits = (rng.standard_normal((n_seq * seq_len, cfg.vocab)) * 0.1).astype(np.float32)
    want_logits, want_grads = _oracle_batch(ref, ids, n_seq, seq_len, dlogits)
    got = m.forward(ids, n_seq, seq_len)
    assert rel_fro(got, want_logits) <= 2e-5
    m.backward(ids, dlogits, n_seq, seq_len)
    assert set(want_grads) == {(l, k) for l in range(cfg.layers) for k in ("q", "v")}
    for (li, kind), (ga, gb) in want_grads.items():
        a, b = m.adapter_grads(li, kind, rank)
        assert rel_fro(a, ga) <= 1e-4, (li, kind, "grad_a")
        assert rel_fro(b, gb) <= 1e-4, (li, kind, "grad_b")


@pytest.mark.gpu
def test_model_longer_sequences_cross_attention_tiles(v):
    """seq_len 150 spans three 64-position tiles (two full, one ragged) and grouped heads (4 query heads on 2
    key/value heads); adapters on all seven projections."""
    ctx = v.GpuContext(0)
    ctx.set_precision(v.PRECISION_FP32_EXACT)
    kw = dict(hidden=256, layers=1, heads=4, kv_heads=2, intermediate=128, vocab=64)
    rank, alpha, n_seq, seq_len = 2, 4.0, 2, 150
    m, ref, cfg = _build(v, ctx, kw, seed=9, rank=rank, alpha=alpha, targets=nl.KINDS)
    rng = np.random.default_rng(1)
    ids = rng.integers(0, cfg.vocab, n_seq * seq_len)
    dlogits = (rng.standard_normal((n_seq * seq_len, cfg.vocab)) * 0.1).astype(np.float32)
    want_logits, want_grads = _oracle_batch(ref, ids, n_seq, seq_len, dlogits)
    assert rel_fro(m.forward(ids, n_seq, seq_len), want_logits) <= 2e-5
    m.backward(ids, dlogits, n_seq, seq_len)
    for (li, kind), (ga, gb) in want_grads.items():
        a, b = m.adapter_grads(li, kind, rank)
        assert rel_fro(a, ga) <= 2e-4 and rel_fro(b, gb) <= 2e-4, (li, kind)


@pytest.mark.gpu
def test_model_tensor_core_path_and_loss(v):
    """bf16 tensor-core linears and LM head: logits within 2e-2, cross-entropy loss within 1e-2 of the oracle,
    gradients within 5e-2 (bf16 operand rounding compounds through the layers)."""
    ctx = v.GpuContext(0)
    ctx.set_precision(v.PRECISION_BF16)
    kw = dict(hidden=128, layers=2, heads=2, kv_heads=1, intermediate=192, vocab=128)
    rank, alpha, n_seq, seq_len = 8, 16.0, 4, 64
    m, ref, cfg = _build(v, ctx, kw, seed=11, rank=rank, alpha=alpha)
    rng = np.random.default_rng(2)
    ids = rng.integers(0, cfg.vocab, n_seq * seq_len)
    targets = rng.integers(0, cfg.vocab, n_seq * seq_len)
    want_logits, _ = _oracle_batch(ref, ids, n_seq, seq_len)
    assert rel_fro(m.forward(ids, n_seq, seq_len), want_logits) <= 2e-2
    # loss = mean over all positions; dlogits = (softmax - onehot) / (n_seq * seq_len)
    losses, dl = [], []
    for s in range(n_seq):
        l, d = nl.softmax_cross_entropy(want_logits[s * seq_len:(s + 1) * seq_len], targets[s * seq_len:(s + 1) * seq_len])
        losses.append(l)
        dl.append(d / n_seq)
    _, want_grads = _oracle_batch(ref, ids, n_seq, seq_len, np.concatenate(dl))
    loss = m.loss_backward(ids, targets, n_seq, seq_len)
    assert abs(loss - float(np.mean(losses))) <= 1e-2 * abs(float(np.mean(losses)))
    for (li, kind), (ga, gb) in want_grads.items():
        a, b = m.adapter_grads(li, kind, rank)
        assert rel_fro(a, ga) <= 5e-2 and rel_fro(b, gb) <= 5e-2, (li, kind, rel_fro(a, ga), rel_fro(b, gb))


@pytest.mark.gpu
def test_model_train_step_reduces_the_loss(v):
    ctx = v.GpuContext(0)
    ctx.set_precision(v.PRECISION_BF16)
    kw = dict(hidden=128, layers=2, heads=2, kv_heads=1, intermediate=192, vocab=128)
    m, ref, cfg = _build(v, ctx, kw, seed=13, rank=8, alpha=16.0)
    opt = v.Adam8bit(v.AdamConfig(lr=5e-3), ctx)
    rng = np.random.default_rng(3)
    n_seq, seq_len = 4, 64
    ids = rng.integers(0, cfg.vocab, n_seq * seq_len)
    targets = np.roll(ids, -1)
    losses = [m.train_step(opt, ids, targets, n_seq, seq_len) for _ in range(40)]
    assert losses[-1] < 0.8 * losses[0], (losses[0], losses[-1])


@pytest.mark.gpu
def test_tensor_core_attention_crosses_tiles_and_sequences(v):
    """bf16 mode runs attention on the tensor cores: 128-query / 128-key tiles forward, 64-key tiles for dQ,
    64-query tiles for dK/dV.  seq_len 300 gives three key tiles with a ragged last one, tiles that run over the
    end of one sequence into the next, and 4 query heads on 2 key/value heads; adapters on q, k, v and o make
    every attention gradient (dQ, dK, dV) reach a checked quantity."""
    ctx = v.GpuContext(0)
    ctx.set_precision(v.PRECISION_BF16)
    kw = dict(hidden=256, layers=2, heads=4, kv_heads=2, intermediate=320, vocab=128)
    rank, alpha, n_seq, seq_len = 8, 16.0, 2, 300
    m, ref, cfg = _build(v, ctx, kw, seed=17, rank=rank, alpha=alpha, targets=("q", "k", "v", "o"))
    rng = np.random.default_rng(4)
    ids = rng.integers(0, cfg.vocab, n_seq * seq_len)
    dlogits = (rng.standard_normal((n_seq * seq_len, cfg.vocab)) * 0.1).astype(np.float32)
    want_logits, want_grads = _oracle_batch(ref, ids, n_seq, seq_len, dlogits)
    assert rel_fro(m.forward(ids, n_seq, seq_len), want_logits) <= 2e-2
    m.backward(ids, dlogits, n_seq, seq_len)
    assert len(want_grads) == 2 * 4
    for (li, kind), (ga, gb) in want_grads.items():
        a, b = m.adapter_grads(li, kind, rank)
        assert rel_fro(a, ga) <= 5e-2 and rel_fro(b, gb) <= 5e-2, (li, kind, rel_fro(a, ga), rel_fro(b, gb))


@pytest.mark.gpu
@pytest.mark.parametrize("n_seq,seq_len", [(3, 40), (1, 129), (5, 64), (2, 1000)])
def test_tensor_core_attention_short_and_odd_sequences(v, n_seq, seq_len):
    """Sequences shorter than one tile (40), one position past a tile (129: the second query tile holds a single
    row), an odd number of sequences, and 1000 positions (eight query tiles, up to eight key tiles each, ragged
    end): the padded row statistics and the zero-filled tile tails must not leak into any gradient."""
    ctx = v.GpuContext(0)
    ctx.set_precision(v.PRECISION_BF16)
    kw = dict(hidden=128, layers=1, heads=2, kv_heads=1, intermediate=192, vocab=96)
    rank, alpha = 4, 8.0
    m, ref, cfg = _build(v, ctx, kw, seed=23 + seq_len, rank=rank, alpha=alpha, targets=("q", "k", "v", "o"))
    rng = np.random.default_rng(seq_len)
    ids = rng.integers(0, cfg.vocab, n_seq * seq_len)
    dlogits = (rng.standard_normal((n_seq * seq_len, cfg.vocab)) * 0.1).astype(np.float32)
    want_logits, want_grads = _oracle_batch(ref, ids, n_seq, seq_len, dlogits)
    assert rel_fro(m.forward(ids, n_seq, seq_len), want_logits) <= 2e-2
    m.backward(ids, dlogits, n_seq, seq_len)
    for (li, kind), (ga, gb) in want_grads.items():
        a, b = m.adapter_grads(li, kind, rank)
        assert np.all(np.isfinite(a)) and np.all(np.isfinite(b))
        assert rel_fro(a, ga) <= 5e-2 and rel_fro(b, gb) <= 5e-2, (li, kind, rel_fro(a, ga), rel_fro(b, gb))


@pytest.mark.gpu
def test_training_steps_are_bitwise_reproducible(v):
    """Two models built from the same numbers take the same three steps: kernels that overlap (parallel lanes,
    side streams, dependent launches) and sums over CTAs (split contractions, per-head dK / dV partials) must not
    make the result depend on timing."""
    kw = dict(hidden=256, layers=2, heads=4, kv_heads=2, intermediate=320, vocab=128)
    rank, alpha, n_seq, seq_len = 8, 16.0, 3, 200
    rng = np.random.default_rng(9)
    ids = rng.integers(0, kw["vocab"], n_seq * seq_len)
    targets = np.roll(ids, -1)
    results = []
    for _ in range(2):
        ctx = v.GpuContext(0)
        ctx.set_precision(v.PRECISION_BF16)
        m, ref, cfg = _build(v, ctx, kw, seed=29, rank=rank, alpha=alpha, targets=("q", "k", "v", "o"))
        opt = v.Adam8bit(v.AdamConfig(lr=1e-3), ctx)
        losses = [m.train_step(opt, ids, targets, n_seq, seq_len) for _ in range(3)]
        weights = [m.adapter_weights(li, k, rank) for li in range(cfg.layers) for k in ("q", "k", "v", "o")]
        results.append((losses, weights))
    assert results[0][0] == results[1][0]
    for (a0, b0), (a1, b1) in zip(results[0][1], results[1][1]):
        assert np.array_equal(a0, a1) and np.array_equal(b0, b1)


@pytest.mark.gpu
def test_model_tf32_mode(v):
    """TF32 precision: fp32 activations between the kernels, fp32 attention, every linear on the tensor cores in
    tf32 (the LM head takes the bf16 tensor-core GEMM, as in bf16 mode)."""
    ctx = v.GpuContext(0)
    ctx.set_precision(v.PRECISION_TF32)
    kw = dict(hidden=128, layers=2, heads=2, kv_heads=1, intermediate=192, vocab=128)
    rank, alpha, n_seq, seq_len = 8, 16.0, 2, 150
    m, ref, cfg = _build(v, ctx, kw, seed=41, rank=rank, alpha=alpha)
    rng = np.random.default_rng(6)
    ids = rng.integers(0, cfg.vocab, n_seq * seq_len)
    dlogits = (rng.standard_normal((n_seq * seq_len, cfg.vocab)) * 0.1).astype(np.float32)
    want_logits, want_grads = _oracle_batch(ref, ids, n_seq, seq_len, dlogits)
    assert rel_fro(m.forward(ids, n_seq, seq_len), want_logits) <= 1e-2
    m.backward(ids, dlogits, n_seq, seq_len)
    for (li, kind), (ga, gb) in want_grads.items():
        a, b = m.adapter_grads(li, kind, rank)
        assert rel_fro(a, ga) <= 2e-2 and rel_fro(b, gb) <= 2e-2, (li, kind, rel_fro(a, ga), rel_fro(b, gb))


@pytest.mark.gpu
def test_model_auto_mode_with_an_ineligible_projection(v):
    """AUTO precision with an MLP width that is no multiple of 64: the raw gate / up matrices take the exact fp32
    path, the quantised down projection the tensor cores through its padded copy, the other projections the fused
    tensor-core kernels; the model runs the fp32-activation pipeline with the tensor-core attention fed through
    conversions (fp32 attention output, fp32 dQ / dK / dV)."""
    ctx = v.GpuContext(0)   # AUTO is the default
    kw = dict(hidden=128, layers=2, heads=2, kv_heads=1, intermediate=200, vocab=128)
    rank, alpha, n_seq, seq_len = 8, 16.0, 2, 150
    m, ref, cfg = _build(v, ctx, kw, seed=43, rank=rank, alpha=alpha, targets=("q", "k", "v", "o", "down"))
    rng = np.random.default_rng(8)
    ids = rng.integers(0, cfg.vocab, n_seq * seq_len)
    targets = rng.integers(0, cfg.vocab, n_seq * seq_len)
    want_logits, _ = _oracle_batch(ref, ids, n_seq, seq_len)
    assert rel_fro(m.forward(ids, n_seq, seq_len), want_logits) <= 2e-2
    losses, dl = [], []
    for s in range(n_seq):
        l, d = nl.softmax_cross_entropy(want_logits[s * seq_len:(s + 1) * seq_len], targets[s * seq_len:(s + 1) * seq_len])
        losses.append(l)
        dl.append(d / n_seq)
    _, want_grads = _oracle_batch(ref, ids, n_seq, seq_len, np.concatenate(dl))
    loss = m.loss_backward(ids, targets, n_seq, seq_len)
    assert abs(loss - float(np.mean(losses))) <= 1e-2 * abs(float(np.mean(losses)))
    for (li, kind), (ga, gb) in want_grads.items():
        a, b = m.adapter_grads(li, kind, rank)
        assert rel_fro(a, ga) <= 5e-2 and rel_fro(b, gb) <= 5e-2, (li, kind, rel_fro(a, ga), rel_fro(b, gb))


@pytest.mark.gpu
def test_precision_can_change_between_calls(v):
    """The activation storage and the row-statistics layout depend on the precision mode; switching the context's
    precision between calls must rebuild them (exact -> bf16 -> exact on one model)."""
    ctx = v.GpuContext(0)
    kw = dict(hidden=128, layers=2, heads=2, kv_heads=1, intermediate=192, vocab=96)
    rank, alpha, n_seq, seq_len = 4, 8.0, 2, 70
    ctx.set_precision(v.PRECISION_FP32_EXACT)
    m, ref, cfg = _build(v, ctx, kw, seed=47, rank=rank, alpha=alpha)
    rng = np.random.default_rng(10)
    ids = rng.integers(0, cfg.vocab, n_seq * seq_len)
    dlogits = (rng.standard_normal((n_seq * seq_len, cfg.vocab)) * 0.1).astype(np.float32)
    want_logits, want_grads = _oracle_batch(ref, ids, n_seq, seq_len, dlogits)
    for mode, tol_l, tol_g in ((v.PRECISION_FP32_EXACT, 2e-5, 2e-4), (v.PRECISION_BF16, 2e-2, 5e-2),
                               (v.PRECISION_FP32_EXACT, 2e-5, 2e-4)):
        ctx.set_precision(mode)
        assert rel_fro(m.forward(ids, n_seq, seq_len), want_logits) <= tol_l
        m.backward(ids, dlogits, n_seq, seq_len)
        for (li, kind), (ga, gb) in want_grads.items():
            a, b = m.adapter_grads(li, kind, rank)
            assert rel_fro(a, ga) <= tol_g and rel_fro(b, gb) <= tol_g, (mode, li, kind, rel_fro(a, ga), rel_fro(b, gb))


@pytest.mark.gpu
def test_batch_shape_can_change_between_calls(v):
    """Fewer sequences reuse the activation storage, more sequences or another length rebuild it."""
    ctx = v.GpuContext(0)
    ctx.set_precision(v.PRECISION_BF16)
    kw = dict(hidden=128, layers=1, heads=2, kv_heads=1, intermediate=192, vocab=96)
    rank, alpha = 4, 8.0
    m, ref, cfg = _build(v, ctx, kw, seed=53, rank=rank, alpha=alpha, targets=("q", "k", "v"))
    rng = np.random.default_rng(12)
    for n_seq, seq_len in ((3, 100), (1, 100), (4, 100), (2, 37), (3, 100)):
        ids = rng.integers(0, cfg.vocab, n_seq * seq_len)
        dlogits = (rng.standard_normal((n_seq * seq_len, cfg.vocab)) * 0.1).astype(np.float32)
        want_logits, want_grads = _oracle_batch(ref, ids, n_seq, seq_len, dlogits)
        assert rel_fro(m.forward(ids, n_seq, seq_len), want_logits) <= 2e-2
        m.backward(ids, dlogits, n_seq, seq_len)
        for (li, kind), (ga, gb) in want_grads.items():
            a, b = m.adapter_grads(li, kind, rank)
            assert rel_fro(a, ga) <= 5e-2 and rel_fro(b, gb) <= 5e-2, (n_seq, seq_len, kind, rel_fro(a, ga), rel_fro(b, gb))


@pytest.mark.gpu
def test_merged_gate_up_layer_equals_the_two_layers(v):
    """MLP width 256 at hidden 128: gate holds 32 768 = 2 x 16 384 elements, so the NF4 payload of gate and up one
    after the other is the payload of the (2I, h) matrix and the bf16 pipeline runs them as ONE layer (one forward
    GEMM, one input-gradient GEMM over both contractions).  A second model with the same weights gets an adapter
    with B = 0 on `up`, which keeps gate and up as two layers: its logits must be bit-identical (every output
    element accumulates the same products in the same order) and its q / v gradients agree to the bf16 rounding of
    the two input gradients that the merged layer no longer rounds separately.  Both also match the oracle."""
    kw = dict(hidden=128, layers=2, heads=2, kv_heads=1, intermediate=256, vocab=128)
    rank, alpha, n_seq, seq_len = 8, 16.0, 2, 150
    rng = np.random.default_rng(12)
    ids = rng.integers(0, kw["vocab"], n_seq * seq_len)
    dlogits = (rng.standard_normal((n_seq * seq_len, kw["vocab"])) * 0.1).astype(np.float32)
    ctx = v.GpuContext(0)
    ctx.set_precision(v.PRECISION_BF16)
    merged, ref, cfg = _build(v, ctx, kw, seed=47, rank=rank, alpha=alpha)
    separate, _, _ = _build(v, ctx, kw, seed=47, rank=rank, alpha=alpha)
    for li in range(cfg.layers):
        a = (rng.standard_normal((4, kw["hidden"])) * 0.1).astype(np.float32)
        separate.attach_adapter(li, "up", a, np.zeros((kw["intermediate"], 4), np.float32), 4, 8.0)
    want_logits, want_grads = _oracle_batch(ref, ids, n_seq, seq_len, dlogits)
    got_m, got_s = merged.forward(ids, n_seq, seq_len), separate.forward(ids, n_seq, seq_len)
    assert np.array_equal(got_m, got_s)
    assert rel_fro(got_m, want_logits) <= 2e-2
    merged.backward(ids, dlogits, n_seq, seq_len)
    separate.backward(ids, dlogits, n_seq, seq_len)
    for (li, kind), (ga, gb) in want_grads.items():
        am, bm = merged.adapter_grads(li, kind, rank)
        as_, bs = separate.adapter_grads(li, kind, rank)
        assert rel_fro(am, as_) <= 1e-2 and rel_fro(bm, bs) <= 1e-2, (li, kind, rel_fro(am, as_), rel_fro(bm, bs))
        assert rel_fro(am, ga) <= 5e-2 and rel_fro(bm, gb) <= 5e-2, (li, kind, rel_fro(am, ga), rel_fro(bm, gb))


def _qkv_case(v, out_path=None):
    """Logits and q / v adapter gradients of a small model on the bf16 pipeline (a fixed seeded case)."""
    kw = dict(hidden=128, layers=2, heads=2, kv_heads=1, intermediate=256, vocab=128)
    rank, alpha, n_seq, seq_len = 8, 16.0, 2, 150
    rng = np.random.default_rng(21)
    ids = rng.integers(0, kw["vocab"], n_seq * seq_len)
    dlogits = (rng.standard_normal((n_seq * seq_len, kw["vocab"])) * 0.1).astype(np.float32)
    ctx = v.GpuContext(0)
    ctx.set_precision(v.PRECISION_BF16)
    m, ref, cfg = _build(v, ctx, kw, seed=53, rank=rank, alpha=alpha)
    out = {"logits": m.forward(ids, n_seq, seq_len)}
    m.backward(ids, dlogits, n_seq, seq_len)
    for li in range(cfg.layers):
        for kind in ("q", "v"):
            out[f"ga_{li}_{kind}"], out[f"gb_{li}_{kind}"] = m.adapter_grads(li, kind, rank)
    if out_path:
        np.savez(out_path, **out)
    return out, (ref, ids, n_seq, seq_len, dlogits)


@pytest.mark.gpu
def test_merged_qkv_layer_equals_the_three_layers(v, tmp_path):
    """q, k and v run as ONE layer in the bf16 pipeline (codes side by side, fp32 block scales decoded from the three
    payloads, the adapters of q and v stacked into one rank-16 adapter with zero blocks).  The same case computed by
    a second process with QLC_LLAMA_NO_QKV=1 (three layers, three GEMMs each way): logits bit-identical (the zero
    blocks add exact zeros), adapter gradients equal up to the bf16 rounding of the three input gradients that the
    merged layer sums in one accumulator; both within the usual bounds of the oracle."""
    import os
    import subprocess
    import sys
    here = os.path.dirname(os.path.abspath(__file__))
    path = str(tmp_path / "separate.npz")
    env = dict(os.environ, QLC_LLAMA_NO_QKV="1")
    code = ("import sys; sys.path.insert(0, %r); sys.path.insert(0, %r); import vkqlora.rs_b200 as v; "
            "import test_gpu_llama as t; t._qkv_case(v, %r)") % (os.path.dirname(here), here, path)
    subprocess.run([sys.executable, "-c", code], check=True, env=env, timeout=300)
    merged, (ref, ids, n_seq, seq_len, dlogits) = _qkv_case(v)
    with np.load(path) as sep:
        assert np.array_equal(merged["logits"], sep["logits"])
        for k in merged:
            if k != "logits":
                assert rel_fro(merged[k], sep[k]) <= 1e-2, (k, rel_fro(merged[k], sep[k]))
    want_logits, want_grads = _oracle_batch(ref, ids, n_seq, seq_len, dlogits)
    assert rel_fro(merged["logits"], want_logits) <= 2e-2
    for (li, kind), (ga, gb) in want_grads.items():
        assert rel_fro(merged[f"ga_{li}_{kind}"], ga) <= 5e-2 and rel_fro(merged[f"gb_{li}_{kind}"], gb) <= 5e-2, (li, kind)


@pytest.mark.gpu
def test_adapters_with_different_scales_keep_three_layers(v):
    """q and v adapters with different alpha / r cannot share one merged adapter: the block keeps q, k and v as three
    layers (and still merges gate / up), and matches the oracle as before."""
    from vkqlora.rs_b200 import llama
    kw = dict(hidden=128, layers=2, heads=2, kv_heads=1, intermediate=256, vocab=128)
    rank, n_seq, seq_len = 8, 2, 150
    ocfg = nl.LlamaConfig(**kw)
    ref = nl.random_model(ocfg, seed=59, targets=("q", "v"), rank=rank, alpha=16.0, scale=0.08)
    ctx = v.GpuContext(0)
    ctx.set_precision(v.PRECISION_BF16)
    m = llama.LlamaModel(llama.LlamaConfig(**kw), ref.embed, ref.final_norm, ctx)
    for li, L in enumerate(ref.layers):
        m.set_layer(li, L.attn_norm, L.mlp_norm, {k: L.proj[k].w for k in nl.KINDS})
        L.proj["v"].alpha = 24.0     # alpha / r = 3 for v, 2 for q
        for k in ("q", "v"):
            m.attach_adapter(li, k, L.proj[k].a, L.proj[k].b, rank, L.proj[k].alpha)
        for k in nl.KINDS:
            L.proj[k].w = m.dequantized_weight(li, k)
    rng = np.random.default_rng(17)
    ids = rng.integers(0, kw["vocab"], n_seq * seq_len)
    dlogits = (rng.standard_normal((n_seq * seq_len, kw["vocab"])) * 0.1).astype(np.float32)
    want_logits, want_grads = _oracle_batch(ref, ids, n_seq, seq_len, dlogits)
    assert rel_fro(m.forward(ids, n_seq, seq_len), want_logits) <= 2e-2
    m.backward(ids, dlogits, n_seq, seq_len)
    for (li, kind), (ga, gb) in want_grads.items():
        a, b = m.adapter_grads(li, kind, rank)
        assert rel_fro(a, ga) <= 5e-2 and rel_fro(b, gb) <= 5e-2, (li, kind, rel_fro(a, ga), rel_fro(b, gb))
