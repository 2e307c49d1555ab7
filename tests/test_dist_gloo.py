"""World-size-2 test (gloo, CPU) of the multi-GPU scheme: rows sharded over ranks, LoRA gradients
summed with one all-reduce, Y / dX slices needing no exchange.  The per-shard arithmetic is done by the
CPU oracle, so this checks the host-side sharding and reduction logic only."""
import os
import socket
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, q):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from oracle import c_oracle as orc
    from refdata import normal
    from vkqlora.rs_b200.dist import allreduce_lora_grads, shard_rows

    out_dim, in_dim, r, batch, alpha = 24, 40, 3, 11, 6.0
    w, a, b = normal(1, out_dim * in_dim, 0.05), normal(2, r * in_dim, 0.2), normal(3, out_dim * r, 0.1)
    x, dy = normal(4, batch * in_dim).reshape(batch, in_dim), normal(5, batch * out_dim).reshape(batch, out_dim)
    wd = orc.quantize_nf4(w, out_dim, in_dim).dequantize()
    lo, hi = shard_rows(batch, rank, world)
    xs, dys = x[lo:hi].reshape(-1), dy[lo:hi].reshape(-1)
    y = orc.qlora_forward(xs, hi - lo, wd, out_dim, in_dim, a, b, r, alpha)
    gx, ga, gb = orc.qlora_backward(xs, dys, hi - lo, wd, out_dim, in_dim, a, b, r, alpha)
    bucket = torch.from_numpy(np.concatenate([ga, gb]))
    allreduce_lora_grads(bucket)
    y_full = orc.qlora_forward(x.reshape(-1), batch, wd, out_dim, in_dim, a, b, r, alpha)
    gx_full, ga_full, gb_full = orc.qlora_backward(x.reshape(-1), dy.reshape(-1), batch, wd, out_dim, in_dim, a, b, r, alpha)
    ok = (np.array_equal(y, y_full.reshape(batch, out_dim)[lo:hi].reshape(-1))        # rows are independent: exact
          and np.array_equal(gx, gx_full.reshape(batch, in_dim)[lo:hi].reshape(-1))
          and np.allclose(bucket.numpy(), np.concatenate([ga_full, gb_full]), rtol=1e-5, atol=1e-6))
    q.put((rank, bool(ok), (lo, hi)))
    dist.destroy_process_group()


def test_row_sharding_and_grad_allreduce_two_ranks():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = sorted(q.get(timeout=120) for _ in procs)
    for p in procs:
        p.join(timeout=60)
    assert [r[1] for r in res] == [True, True], res
    assert res[0][2] == (0, 6) and res[1][2] == (6, 11)


def test_shard_rows_covers_everything():
    from vkqlora.rs_b200.dist import shard_rows

    for total in (0, 1, 7, 8192, 65536):
        for world in (1, 2, 3, 8):
            spans = [shard_rows(total, r, world) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == total
            assert all(spans[i][1] == spans[i + 1][0] for i in range(world - 1))
            assert max(e - b for b, e in spans) - min(e - b for b, e in spans) <= 1
    with pytest.raises(ValueError):
        shard_rows(10, 2, 2)


def _col_worker(rank, world, port, q):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from oracle import c_oracle as orc
    from refdata import normal
    from vkqlora.rs_b200.dist import column_shard_weights

    out_dim, in_dim, r, batch, alpha = 768, 64, 4, 5, 8.0   # three 256-row units over two ranks: 512 + 256
    w, a, b = normal(1, out_dim * in_dim, 0.05), normal(2, r * in_dim, 0.2), normal(3, out_dim * r, 0.1)
    x, dy = normal(4, batch * in_dim), normal(5, batch * out_dim).reshape(batch, out_dim)
    ws, a_s, bs, lo, hi = column_shard_weights(w, a, b, out_dim, in_dim, r, rank, world)
    n_loc = hi - lo
    q_loc = orc.quantize_nf4(ws, n_loc, in_dim)
    q_full = orc.quantize_nf4(w, out_dim, in_dim)
    # the shard's quantisation is the slice of the whole tensor's: same codes, same 8-bit scales
    same_q = (np.array_equal(q_loc.codes, q_full.codes[lo * in_dim // 2:hi * in_dim // 2])
              and np.array_equal(q_loc.absmax_codes, q_full.absmax_codes[lo * in_dim // 64:hi * in_dim // 64])
              and np.array_equal(q_loc.dequantize(), q_full.dequantize().reshape(out_dim, in_dim)[lo:hi].reshape(-1)))
    y_loc = orc.qlora_forward(x, batch, q_loc.dequantize(), n_loc, in_dim, a_s, bs, r, alpha)
    _, _, gb_loc = orc.qlora_backward(x, dy[:, lo:hi].reshape(-1), batch, q_loc.dequantize(), n_loc, in_dim, a_s, bs, r, alpha)
    y_full = orc.qlora_forward(x, batch, q_full.dequantize(), out_dim, in_dim, a, b, r, alpha).reshape(batch, out_dim)
    _, _, gb_full = orc.qlora_backward(x, dy.reshape(-1), batch, q_full.dequantize(), out_dim, in_dim, a, b, r, alpha)
    ok = (same_q and np.array_equal(y_loc.reshape(batch, n_loc), y_full[:, lo:hi])     # columns are independent: exact
          and np.array_equal(gb_loc, gb_full.reshape(out_dim, r)[lo:hi].reshape(-1)))
    # the only "exchange" is the concatenation of the output slices by whoever consumes Y (here: an all_gather
    # of equal-sized padded slices, to show that the pieces tile the full result)
    pad = torch.zeros(batch, 512)
    pad[:, :n_loc] = torch.from_numpy(y_loc.reshape(batch, n_loc))
    parts = [torch.zeros(batch, 512) for _ in range(world)]
    dist.all_gather(parts, pad)
    y_cat = torch.cat([parts[0][:, :512], parts[1][:, :256]], dim=1).numpy()
    ok = ok and np.array_equal(y_cat, y_full)
    q.put((rank, bool(ok), (lo, hi)))
    dist.destroy_process_group()


def test_column_sharding_needs_no_collective_two_ranks():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_col_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = sorted(q.get(timeout=120) for _ in procs)
    for p in procs:
        p.join(timeout=60)
    assert [r[1] for r in res] == [True, True], res
    assert res[0][2] == (0, 512) and res[1][2] == (512, 768)


def test_shard_cols_covers_everything_on_tile_boundaries():
    from vkqlora.rs_b200.dist import shard_cols

    for out_dim in (256, 4096, 11008, 1000, 100):
        for world in (1, 2, 3, 8):
            spans = [shard_cols(out_dim, r, world) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == out_dim
            assert all(spans[i][1] == spans[i + 1][0] for i in range(world - 1))
            assert all(b % 256 == 0 for b, e in spans if e > b)  # empty shards sit at the end
