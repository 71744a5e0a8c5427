"""Multi-GPU layouts of the hot path (one process per GPU).

Two ways the path shards:

  * independent sequences: sequence s runs on rank s mod G with a full replica of the packed
    weights; no collective touches the data path (`assign_sequences`).  Throughput is the
    sum over ranks, timed as the maximum over ranks (`max_over_ranks`).
  * one large model, batch 1: every packed matrix is split by OUTPUT columns
    (`column_shard`): rank g keeps columns [g*Mw, min(M, (g+1)*Mw)) of W, mx and rx -- the
    per-row vectors my, ry and the activations stay whole -- computes its slice of every
    matmul and the slices are all-gathered (`gather_columns`, NCCL over NVLink, or gloo on
    CPU in the tests).  The packing is done on the whole matrix first, so codes and scales
    are those of the unsharded model.

The reference has no counterpart: its only multi-device mechanism is placing whole layers
on different devices (rwkv_pip_package/src/rwkv/model.py:684-749).
"""
from __future__ import annotations

import torch
import torch.distributed as dist


def assign_sequences(n_sequences, world, rank):
    """Sequence ids of `rank`: s with s % world == rank."""
    return [s for s in range(n_sequences) if s % world == rank]


def max_over_ranks(values, device=None):
    """Element-wise maximum of a list of floats over all ranks (identity when not distributed)."""
    t = torch.tensor(list(values), dtype=torch.float64, device=device)
    if dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return t.tolist()


def shard_width(M, world):
    """Columns per rank: ceil(M / world) rounded up to 16 (rows of a slice stay 16-byte aligned)."""
    return ((M + world - 1) // world + 15) // 16 * 16


def column_range(M, world, rank):
    mw = shard_width(M, world)
    lo = min(M, rank * mw)
    return lo, min(M, lo + mw)


def column_shard(q, mx, rx, world, rank):
    """Slice a packed matrix (q uint8 [N, M], mx, rx [M]) to the columns of `rank`.  Returns
    contiguous-by-rows copies: q_local [N, m] with a 16-byte row stride, mx_local, rx_local
    [m]; m may be 0 for trailing ranks of a narrow matrix."""
    N, M = q.shape
    lo, hi = column_range(M, world, rank)
    m = hi - lo
    stride = max(16, (m + 15) // 16 * 16)
    buf = torch.zeros((N, stride), dtype=torch.uint8, device=q.device)
    if m > 0:
        buf[:, :m].copy_(q[:, lo:hi])
    return buf[:, :m], mx[lo:hi].contiguous(), rx[lo:hi].contiguous()


def gather_columns(local, M, world, group=None):
    """All-gather per-rank column slices.  `local`: [..., Mw] (Mw = shard_width(M, world), the
    tail beyond a rank's own columns is ignored).  Returns [..., M] in column order."""
    if world == 1:
        return local[..., :M]
    mw = local.shape[-1]
    lead = local.shape[:-1]
    loc = local.contiguous()
    flat = torch.empty(world * loc.numel(), dtype=local.dtype, device=local.device)
    dist.all_gather_into_tensor(flat, loc.reshape(-1), group=group)
    out = flat.view((world,) + tuple(lead) + (mw,))
    if len(lead) == 0:
        return out.reshape(world * mw)[:M]
    perm = list(range(1, len(lead) + 1)) + [0, len(lead) + 1]
    return out.permute(*perm).reshape(*lead, world * mw)[..., :M]
