"""Straggler shedding: the slowest ranks skip their last micro-batch (reference: pure planner ``shed_plan``
round2/source/train.py:14305 and the probe ``ShedS5`` :14345-14483; off in the final recipe and refused with MoE).

The plan is a pure function of the gathered timings so every rank computes the same answer.
"""
from __future__ import annotations

import torch
import torch.distributed as dist


def shed_plan(times_ms, accum: int, threshold: float = 1.08, max_shed_frac: float = 0.25):
    """``times_ms[r]``: rank r's time for its micro-batches.  A rank sheds one micro-batch when it is slower than
    ``threshold`` x median; at most ``max_shed_frac`` of the ranks shed; never below one micro-batch.  Returns the
    micro-batch count per rank and the total so the loss can be re-normalised."""
    n = len(times_ms)
    order = sorted(range(n), key=lambda r: (-times_ms[r], r))
    med = sorted(times_ms)[n // 2]
    budget = int(n * max_shed_frac)
    counts = [accum] * n
    for r in order[:budget]:
        if accum > 1 and times_ms[r] > threshold * med:
            counts[r] = accum - 1
    return counts, sum(counts)


class ShedProbe:
    def __init__(self, rt, accum: int, group=None):
        self.rt, self.accum, self.group = rt, accum, group or rt.control_group
        self.counts = [accum] * rt.world

    def update(self, my_ms: float):
        t = torch.zeros(self.rt.world, dtype=torch.float64)
        t[self.rt.rank] = my_ms
        if self.rt.ddp and self.rt.world > 1:
            dist.all_reduce(t, group=self.group)
        self.counts, total = shed_plan(t.tolist(), self.accum)
        return self.counts[self.rt.rank], total
