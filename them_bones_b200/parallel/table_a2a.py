"""Row-sharded table exchange: lookups and sparse gradients routed to the row owners.

Owner of global row ``r`` is rank ``r % world`` and its local index is ``r // world`` (the reference's host tables use
the same ownership rule and exchange through /dev/shm staging files and barriers, round2/source/train.py:3653-3680).

Two transports with the same interface:

* ``CollectiveExchange`` -- ``all_to_all_single`` on the process group (NCCL on GPUs, gloo on CPU).  This is the baseline
  path and the oracle for the fused one.
* ``PeerExchange`` (``parallel.symm``) -- the rows are read straight out of the owners' shards through NVLink peer
  pointers by one gather kernel, and gradients are pushed into the owners' staging buffers by peer stores; no NCCL call.
"""
from __future__ import annotations

import torch
import torch.distributed as dist


def _bucket(ids: torch.Tensor, world: int):
    """Stable sort of ``ids`` by owner.  Returns ``(order, counts[world])``."""
    owner = ids % world
    order = torch.argsort(owner, stable=True)
    counts = torch.bincount(owner, minlength=world)
    return order, counts


class LocalExchange:
    """world == 1: every row is local."""

    def lookup(self, shard, ids, world):
        return shard.index_select(0, ids)

    def send_grads(self, ids, grads, world):
        return ids, grads

    def all_ok(self, ok):
        return ok


class CollectiveExchange:
    def __init__(self, group, world: int, rank: int, device):
        self.group, self.world, self.rank, self.device = group, world, rank, device

    def _counts(self, counts):
        recv = torch.empty_like(counts)
        dist.all_to_all_single(recv, counts, group=self.group)
        return recv

    def _a2a(self, x, send_counts, recv_counts):
        out = x.new_empty((int(recv_counts.sum()),) + tuple(x.shape[1:]))
        dist.all_to_all_single(out, x.contiguous(), output_split_sizes=recv_counts.tolist(),
                               input_split_sizes=send_counts.tolist(), group=self.group)
        return out

    def lookup(self, shard, ids, world):
        order, counts = _bucket(ids, world)
        recv_counts = self._counts(counts)
        want = self._a2a((ids[order] // world), counts, recv_counts)         # local row ids requested of me
        rows = shard.index_select(0, want)
        back = self._a2a(rows, recv_counts, counts)                         # rows for my requests, owner-sorted
        out = torch.empty_like(back)
        out[order] = back
        return out

    def send_grads(self, ids, grads, world):
        order, counts = _bucket(ids, world)
        recv_counts = self._counts(counts)
        lids = self._a2a(ids[order] // world, counts, recv_counts)
        lgrads = self._a2a(grads[order], counts, recv_counts)
        return lids, lgrads

    def all_ok(self, ok):
        t = ok.to(torch.int32).reshape(1).clone()
        dist.all_reduce(t, op=dist.ReduceOp.MIN, group=self.group)
        return t[0] > 0


def make_exchange(group, world: int, rank: int, device):
    if world == 1:
        return LocalExchange()
    return CollectiveExchange(group, world, rank, device)
