"""Launch/runtime layer: device choice, process group, seeding, device timers.

Reference behaviour (round2/source/train.py:3157-3216): ``detect_device_type`` prefers the accelerator,
``init_runtime`` seeds, creates the process group (``nccl`` with ``device_id`` on CUDA, ``gloo`` on CPU) and
barriers; compute dtype is bf16 on accelerators and fp32 on CPU.  One process drives one GPU.
"""
from __future__ import annotations

import os
import time
from dataclasses import dataclass

import torch
import torch.distributed as dist


def get_dist_info():
    """``(ddp, rank, local_rank, world_size)`` from the torchrun environment."""
    if "RANK" in os.environ and "WORLD_SIZE" in os.environ:
        return True, int(os.environ["RANK"]), int(os.environ.get("LOCAL_RANK", 0)), int(os.environ["WORLD_SIZE"])
    return False, 0, 0, 1


def print0(*args, **kw):
    if int(os.environ.get("RANK", 0)) == 0:
        print(*args, **kw, flush=True)


def detect_device_type() -> str:
    forced = os.environ.get("BONES_DEVICE")
    if forced:
        return forced
    return "cuda" if torch.cuda.is_available() else "cpu"


@dataclass
class Runtime:
    ddp: bool
    rank: int
    local_rank: int
    world: int
    device: torch.device
    device_type: str
    control_group: object = None      # gloo group for host-side control (never queues behind device collectives)

    @property
    def is_master(self) -> bool:
        return self.rank == 0


def init_runtime(device_type: str | None = None, seed: int = 42) -> Runtime:
    device_type = device_type or detect_device_type()
    ddp, rank, local_rank, world = get_dist_info()
    torch.manual_seed(seed)
    if device_type == "cuda":
        device = torch.device("cuda", local_rank)
        torch.cuda.set_device(device)
        torch.cuda.manual_seed(seed)
    else:
        device = torch.device("cpu")
    control = None
    if ddp and not dist.is_initialized():
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29500")
        if device_type == "cuda":
            dist.init_process_group("nccl", device_id=device)
        else:
            dist.init_process_group("gloo")
    if ddp:
        if device_type == "cuda":
            control = dist.new_group(backend="gloo")
        dist.barrier()
    return Runtime(ddp, rank, local_rank, world, device, device_type, control)


def cleanup_runtime():
    if dist.is_available() and dist.is_initialized():
        dist.destroy_process_group()


def synchronize(device_type: str):
    if device_type == "cuda":
        torch.cuda.synchronize()


def compute_dtype_for(device_type: str) -> torch.dtype:
    return torch.bfloat16 if device_type == "cuda" else torch.float32


class StepTimer:
    """Device-side step timer: CUDA events on the launching stream, reduced as the max over ranks.  On CPU it is a
    wall clock.  Replaces the competition kit's ``record_step_boundary``."""

    def __init__(self, rt: Runtime):
        self.rt = rt
        self.cuda = rt.device_type == "cuda"
        self._t0 = None
        self._ev = None

    def start(self):
        if self.cuda:
            self._ev = (torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
            self._ev[0].record()
        else:
            self._t0 = time.perf_counter()

    def stop(self) -> float:
        """Milliseconds since ``start`` (max over ranks).  Synchronises."""
        if self.cuda:
            self._ev[1].record()
            self._ev[1].synchronize()
            ms = self._ev[0].elapsed_time(self._ev[1])
        else:
            ms = (time.perf_counter() - self._t0) * 1e3
        return max_over_ranks(ms, self.rt)


def max_over_ranks(value: float, rt: Runtime) -> float:
    if not rt.ddp or rt.world == 1:
        return float(value)
    t = torch.tensor([float(value)], dtype=torch.float64,
                     device=rt.device if rt.device_type == "cuda" else "cpu")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())
