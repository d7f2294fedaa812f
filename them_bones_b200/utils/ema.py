"""Tail averaging of the weights (reference: ``EmaLawa`` round2/source/train.py:13462; round 1's tail blend
``theta_T + g (theta_T - theta_ref)``, round1/source/train.py:10091)."""
from __future__ import annotations

import torch


class EmaLawa:
    def __init__(self, params, start: float, every: int, decay: float = 0.0):
        self.params, self.start, self.every, self.decay = list(params), start, every, decay
        self.avg, self.count = None, 0

    @torch.no_grad()
    def update(self, step: int, progress: float):
        if progress < self.start or step % self.every:
            return False
        if self.avg is None:
            self.avg = [p.detach().float().clone() for p in self.params]
            self.count = 1
            return True
        self.count += 1
        w = (1 - self.decay) if self.decay > 0 else 1.0 / self.count
        for a, p in zip(self.avg, self.params):
            a.lerp_(p.detach().float(), w)
        return True

    @torch.no_grad()
    def swap_in(self):
        if self.avg is not None:
            for a, p in zip(self.avg, self.params):
                p.copy_(a.to(p.dtype))


@torch.no_grad()
def tail_blend(params, ref_params, g: float = -0.075):
    for p, r in zip(params, ref_params):
        p.add_(g * (p - r.to(p.device, p.dtype)))
