"""Multi-GPU plumbing for the QloraLinear path: token rows are sharded across ranks (one process per
GPU), the quantised weight and the adapter are replicated, and the only exchange step is a sum
all-reduce of the concatenated LoRA gradients (grad_a followed by grad_b).

The reference has no multi-device path; the only behaviour to preserve is that grad_a / grad_b are the
sums over *all* token rows (qlora-core/src/qlora.rs:147,151 contract over the batch), which a sum over
ranks of per-shard gradients reproduces up to fp32 summation order.
"""
from __future__ import annotations

from typing import Tuple

import numpy as np


def shard_rows(total_rows: int, rank: int, world: int) -> Tuple[int, int]:
    """[begin, end) of the token rows owned by `rank`: contiguous, sizes differ by at most one."""
    if world <= 0 or not (0 <= rank < world):
        raise ValueError(f"bad rank/world: {rank}/{world}")
    base, rem = divmod(total_rows, world)
    begin = rank * base + min(rank, rem)
    return begin, begin + base + (1 if rank < rem else 0)


def allreduce_lora_grads(bucket, group=None):
    """Sums the contiguous grad_a‖grad_b bucket (a torch tensor on this rank's device, or on the CPU
    for gloo) over all ranks, in place.  No averaging: loss scaling lives in dY, as in the reference."""
    import torch.distributed as dist

    if dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.all_reduce(bucket, op=dist.ReduceOp.SUM, group=group)
    return bucket


# ---- column (out_dim) sharding: no collective ---------------------------------------------------------------------
# Output features are independent in Y = X·deq(W)^T + s·(X·A^T)·B^T (qlora-core/src/lora.rs:169-183 computes one
# output column at a time): rank g keeps rows [begin, end) of W (quantised on their own) and of B, and all of A,
# and produces Y[:, begin:end] - and grad_B[begin:end] = (s·dY[:, begin:end])^T·(X·A^T) - without talking to anyone.
# dX and grad_A contract over out_dim and would need a sum over ranks, so this mode is for layers whose input
# gradient is not needed (inference, or the first layer); training layers shard token rows instead (above).

COL_SHARD_MULTIPLE = 256  # rows of W per shard boundary: the GEMM's column tile, and with in_dim a multiple of 64 it
#                           keeps every double-quantisation group (16 384 weights) inside one shard


def shard_cols(out_dim: int, rank: int, world: int, multiple: int = COL_SHARD_MULTIPLE) -> Tuple[int, int]:
    """[begin, end) of the output features owned by `rank`: contiguous, boundaries on multiples of `multiple`
    (the last shard takes the remainder), sizes as even as that allows."""
    if world <= 0 or not (0 <= rank < world):
        raise ValueError(f"bad rank/world: {rank}/{world}")
    units = -(-out_dim // multiple)  # ceil
    base, rem = divmod(units, world)
    b_units = rank * base + min(rank, rem)
    e_units = b_units + base + (1 if rank < rem else 0)
    return min(b_units * multiple, out_dim), min(e_units * multiple, out_dim)


def column_shard_weights(w, a, b, out_dim: int, in_dim: int, r: int, rank: int, world: int,
                         multiple: int = COL_SHARD_MULTIPLE):
    """This rank's part of a layer for the column-sharded mode: (W[begin:end, :], A, B[begin:end, :], begin, end) as
    flat float32 arrays.  Quantising the W slice gives exactly the codes and scales of the same rows of the
    whole tensor when begin * in_dim is a multiple of the double-quantisation group (16 384 weights): true for
    the default `multiple` and any in_dim that is a multiple of 64."""
    begin, end = shard_cols(out_dim, rank, world, multiple)
    w2 = np.ascontiguousarray(w, np.float32).reshape(out_dim, in_dim)
    b2 = np.ascontiguousarray(b, np.float32).reshape(out_dim, r)
    return (w2[begin:end].reshape(-1).copy(), np.ascontiguousarray(a, np.float32).reshape(-1), b2[begin:end].reshape(-1).copy(),
            begin, end)
