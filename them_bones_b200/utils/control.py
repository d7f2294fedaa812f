"""Step control: collective health/stop decisions, the predictive stop rule and the asynchronous step boundary.

Reference: every step the vector ``[bad_loss, stop, rank0_clock_ms]`` is MAX-all-reduced so that no rank starts another
step alone and all ranks leave together on a bad loss (round2/source/train.py:22959-22983); it runs on its own gloo
group so host control never queues behind device collectives (:21810-21893).  The stop rule predicts whether one more
step fits: ``elapsed + max(last 20 dt) + reserve >= budget`` (:22945-22958).  The asynchronous boundary (``BoundaryS11``,
:14064-14118) reads the loss with a non-blocking device-to-host copy into pinned memory plus an event, and evaluates a
step's tail one step late, with a forced synchronous boundary every ``sync_every`` steps so a latent device error
surfaces within that many steps.
"""
from __future__ import annotations

import collections
import math
import time

import torch
import torch.distributed as dist


class StepControl:
    def __init__(self, rt, bad_loss: float = 100.0):
        self.rt, self.bad_loss = rt, bad_loss
        self.group = rt.control_group
        self.dropped = 0                 # test hook: number of control messages to drop (host-side fault injection)

    def decide(self, loss_value: float | None, want_stop: bool, clock_ms: float = 0.0):
        """Returns ``(bad, stop, rank0_clock_ms)`` agreed by every rank."""
        bad = loss_value is not None and (math.isnan(loss_value) or loss_value > self.bad_loss)
        vec = torch.tensor([int(bad), int(want_stop), int(clock_ms) if self.rt.rank == 0 else 0], dtype=torch.int64)
        if self.rt.ddp and self.rt.world > 1:
            if self.rt.device_type == "cuda" and self.group is None:
                vec = vec.to(self.rt.device)
            dist.all_reduce(vec, op=dist.ReduceOp.MAX, group=self.group)
        return bool(vec[0]), bool(vec[1]), float(vec[2])


class StopRule:
    def __init__(self, budget_s: float, reserve_s: float = 0.0, window: int = 20):
        self.budget, self.reserve = budget_s, reserve_s
        self.dts = collections.deque(maxlen=window)

    def observe(self, dt_s: float):
        self.dts.append(dt_s)

    def should_stop(self, elapsed_s: float) -> bool:
        if self.budget <= 0:
            return False
        worst = max(self.dts) if self.dts else 0.0
        return elapsed_s + worst + self.reserve >= self.budget


class AsyncBoundary:
    """Loss read-back without a device synchronise in the step loop."""

    def __init__(self, device, sync_every: int = 100):
        self.cuda = torch.device(device).type == "cuda"
        self.sync_every = sync_every
        self.pinned = torch.zeros(2, dtype=torch.float32).pin_memory() if self.cuda else torch.zeros(2)
        self.pending = None              # (step, event, t_host)
        self.waits_ms = 0.0

    def submit(self, step: int, loss: torch.Tensor):
        slot = step % 2
        if self.cuda:
            self.pinned[slot:slot + 1].copy_(loss.detach().reshape(1).float(), non_blocking=True)
            ev = torch.cuda.Event()
            ev.record()
        else:
            self.pinned[slot] = float(loss)
            ev = None
        self.pending = (step, ev, time.perf_counter())

    def must_sync(self, step: int) -> bool:
        return self.sync_every > 0 and step % self.sync_every == 0

    def collect(self):
        """``(step, loss_value)`` of the submitted step (waits on its event only)."""
        if self.pending is None:
            return None
        step, ev, _ = self.pending
        if ev is not None:
            t0 = time.perf_counter()
            ev.synchronize()
            self.waits_ms += (time.perf_counter() - t0) * 1e3
        self.pending = None
        return step, float(self.pinned[step % 2])
