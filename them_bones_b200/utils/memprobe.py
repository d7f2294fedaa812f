"""Memory and latency probes (reference: ``thr2_memory_line`` round2/source/train.py:10026, ``Db4Barrier`` :10053-10089,
``MemPhase`` :10092-10133)."""
from __future__ import annotations

import torch


def memory_line(device) -> str:
    if torch.device(device).type != "cuda":
        return "memory: cpu run"
    s = torch.cuda.memory_stats(device)
    gb = 1 / 2 ** 30
    return (f"memory: allocated {s['allocated_bytes.all.current'] * gb:.2f} GiB (peak "
            f"{s['allocated_bytes.all.peak'] * gb:.2f}), reserved {s['reserved_bytes.all.current'] * gb:.2f} GiB (peak "
            f"{s['reserved_bytes.all.peak'] * gb:.2f}), retries {s.get('num_alloc_retries', 0)}")


class MemPhase:
    """Synchronise at each phase boundary of one chosen step and report peak/held memory per phase."""

    def __init__(self, device, step: int):
        self.device, self.step, self.rows, self.active = torch.device(device), step, [], False

    def begin(self, step: int):
        self.active = step == self.step and self.device.type == "cuda"
        if self.active:
            torch.cuda.synchronize()
            torch.cuda.reset_peak_memory_stats(self.device)

    def mark(self, name: str):
        if not self.active:
            return
        torch.cuda.synchronize()
        gb = 1 / 2 ** 30
        self.rows.append((name, torch.cuda.max_memory_allocated(self.device) * gb,
                          torch.cuda.memory_allocated(self.device) * gb))
        torch.cuda.reset_peak_memory_stats(self.device)

    def report(self) -> str:
        return "; ".join(f"{n}: peak {p:.2f} held {h:.2f} GiB" for n, p, h in self.rows)


class MicroBarrier:
    """Event after each backward so the host never runs more than one micro-step ahead of the device."""

    def __init__(self, device):
        self.cuda = torch.device(device).type == "cuda"
        self.prev = None

    def tick(self):
        if not self.cuda:
            return
        ev = torch.cuda.Event()
        ev.record()
        if self.prev is not None:
            self.prev.synchronize()
        self.prev = ev
