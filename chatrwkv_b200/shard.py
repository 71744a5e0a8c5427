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


class _RawCuda:
    """A span of device memory owned elsewhere, presented through __cuda_array_interface__."""

    def __init__(self, ptr, nbytes):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 3}


class PeerRegion:
    """One region of device memory per rank, laid out identically everywhere and mapped by every
    other rank (CUDA IPC over NVLink): the activation buffers of the column-sharded decode and
    the arrival words of its launches.  `fields` = [(name, dtype, numel)].  `view(name)` is this
    rank's tensor, `peer_ptr(name, other)` the address of the same buffer on rank `other`.

    The matmul kernels store into the peers' regions themselves (rwkv_mm8_one_batch_exchange);
    torch.distributed is used once, here, to pass the 64-byte handles around."""

    FLAG_WORDS = 64

    def __init__(self, fields, device, world, rank, group=None):
        import ctypes as C
        from . import _lib
        L = _lib.lib()
        self.world, self.rank, self.device = world, rank, device
        self.offsets, off = {}, 0
        for name, dtype, numel in fields:
            self.offsets[name] = (off, dtype, numel)
            off += (numel * torch.empty((), dtype=dtype).element_size() + 255) // 256 * 256
        self.flag_off = off
        off += self.FLAG_WORDS * 4
        self.nbytes = (off + 255) // 256 * 256
        with torch.cuda.device(device):
            p = C.c_void_p()
            _lib.check(L.rwkv_peer_alloc(self.nbytes, C.byref(p)), "peer_alloc")
            self.base = p.value
            handle = (C.c_ubyte * _lib.PEER_HANDLE_BYTES)()
            _lib.check(L.rwkv_peer_export(self.base, handle), "peer_export")
            mine = torch.tensor(list(handle), dtype=torch.uint8, device=device)
            allh = torch.empty(world * _lib.PEER_HANDLE_BYTES, dtype=torch.uint8, device=device)
            dist.all_gather_into_tensor(allh, mine, group=group)
            allh = allh.cpu().view(world, -1)
            self.bases = []
            for r in range(world):
                if r == rank:
                    self.bases.append(self.base)
                    continue
                h = (C.c_ubyte * _lib.PEER_HANDLE_BYTES)(*allh[r].tolist())
                q = C.c_void_p()
                _lib.check(L.rwkv_peer_open(h, C.byref(q)), "peer_open")
                self.bases.append(q.value)
            self._bytes = torch.as_tensor(_RawCuda(self.base, self.nbytes), device=device)
        dist.barrier(group=group)
        self.others = [r for r in range(world) if r != rank]
        self.seq = 0

    def view(self, name):
        off, dtype, numel = self.offsets[name]
        es = torch.empty((), dtype=dtype).element_size()
        return self._bytes[off:off + numel * es].view(dtype)

    def peer_ptr(self, name, other, elem_offset=0):
        off, dtype, _ = self.offsets[name]
        return self.bases[other] + off + elem_offset * torch.empty((), dtype=dtype).element_size()

    # arrival words: word r of a rank = sequence number of the last launch of rank r whose results
    # have all arrived there; word FLAG_WORDS-3 = sequence base, FLAG_WORDS-2 = done counter, FLAG_WORDS-1 = error
    def arrived_ptr(self, on_rank, word=0):
        return self.bases[on_rank] + self.flag_off + 4 * word

    # A token's launches are numbered 1..n relative to the device word `seq_base`, which
    # `begin_token` advances by n in stream order: the numbers a launch carries are the same for
    # every token, so a captured graph can be replayed.
    def begin_token(self, n_launches, stream):
        from . import _lib
        self._rel = 0
        self._n = n_launches
        _lib.check(_lib.lib().rwkv_peer_advance(self.arrived_ptr(self.rank, self.FLAG_WORDS - 3), n_launches, stream),
                   "peer_advance")

    def exchange(self, y_names_and_offsets, wait):
        """The rwkv_mm8_exchange of the token's next launch.  `y_names_and_offsets`: per problem
        (buffer name, element offset of its y inside the buffer); `wait`: whether the launch's
        inputs include results of the previous launch of the other ranks."""
        from . import _lib
        e = _lib.Mm8Exchange()
        for z, (name, eo) in enumerate(y_names_and_offsets):
            for i, r in enumerate(self.others):
                e.peer_y[z][i] = self.peer_ptr(name, r, eo)
        e.arrived = self.arrived_ptr(self.rank)
        for i, r in enumerate(self.others):
            e.peer_arrived[i] = self.arrived_ptr(r, self.rank)
        e.done_counter = self.arrived_ptr(self.rank, self.FLAG_WORDS - 2)
        e.error = self.arrived_ptr(self.rank, self.FLAG_WORDS - 1)
        e.seq_base = self.arrived_ptr(self.rank, self.FLAG_WORDS - 3)
        # before the first token seq_base is n (advanced once), so numbers start at n + 1 > 0
        e.wait_seq = self._rel if wait else 0
        self._rel += 1
        e.signal_seq = self._rel
        e.world, e.rank = self.world, self.rank
        return e

    def end_token(self, stream):
        """Enqueue a wait until the results of every rank's last launch have arrived here."""
        from . import _lib
        assert self._rel == self._n, (self._rel, self._n)
        _lib.check(_lib.lib().rwkv_peer_wait(self.arrived_ptr(self.rank), self.world, self._rel,
                                             self.arrived_ptr(self.rank, self.FLAG_WORDS - 3),
                                             self.arrived_ptr(self.rank, self.FLAG_WORDS - 1), stream), "peer_wait")

    def take_error(self):
        torch.cuda.synchronize(self.device)
        w = self._bytes[self.flag_off:self.flag_off + 4 * self.FLAG_WORDS].view(torch.int32)
        e = int(w[self.FLAG_WORDS - 1].item())
        if e:
            w[self.FLAG_WORDS - 1] = 0
        return e
