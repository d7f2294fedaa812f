"""The training engine: model + optimizer + tables + data + one public ``train_step``.

``Trainer.train_step(inputs, targets)`` is the call a user makes per optimizer step (``train.py`` and ``bench.py`` both
go through it): it copies the step's pinned host windows to the device, runs ``grad_accum`` micro-steps of forward /
backward / ``optimizer.accumulate()``, applies the schedules, runs the distributed optimizer step and the table update,
and returns the step's mean loss as a device scalar (reference step loop: round2/source/train.py:22565-23078).
"""
from __future__ import annotations

import time

import torch
import torch.distributed as dist

from . import ops
from .config import GPTConfig, Hyper, switches
from .models.gpt import GPT
from .models.tables import HashedTables
from .optim import schedules
from .optim.muon_adamw import setup_optimizer
from .runtime import Runtime, compute_dtype_for, print0


class Trainer:
    def __init__(self, config: GPTConfig, hyper: Hyper, rt: Runtime, *, device_batch: int | None = None,
                 total_batch: int | None = None, optimizer_kind: str | None = None, fused_comm: bool | None = None,
                 horizon_steps: int = 0, budget_seconds: float = 0.0, init_state: dict | None = None):
        sw = switches()
        self.config, self.hyper, self.rt = config, hyper, rt
        self.dtype = compute_dtype_for(rt.device_type)
        self.device_batch = device_batch or hyper.device_batch
        self.total_batch = total_batch or hyper.total_batch
        tokens_per_micro = self.device_batch * config.sequence_len * rt.world
        if self.total_batch % tokens_per_micro:
            raise ValueError(f"total batch {self.total_batch} is not a multiple of {tokens_per_micro} tokens per micro-step")
        self.grad_accum = self.total_batch // tokens_per_micro
        self.local_windows = self.device_batch * self.grad_accum
        self.horizon_steps, self.budget_seconds = horizon_steps, budget_seconds
        ep_group = dist.group.WORLD if (rt.ddp and config.moe_layers) else None
        torch.manual_seed(hyper.seed)
        model = GPT(config, ep_group=ep_group, ep_world=rt.world if config.moe_layers else 1,
                    ep_rank=rt.rank if config.moe_layers else 0)
        model.init_weights(hyper.seed)
        if init_state is not None:                 # resume: a checkpoint's ``model_state`` replaces the fresh weights
            from .utils.ckpt import load_model_state
            load_model_state(model, init_state, ep_world=rt.world if config.moe_layers else 1,
                             ep_rank=rt.rank if config.moe_layers else 0)
        model = model.to(rt.device)
        model.cast_compute(self.dtype)
        self.model = model
        self.comm = None
        use_fused = sw["FUSED_COMM"] if fused_comm is None else fused_comm
        extras = dict(grad_clip=sw["GRAD_CLIP"], bf16_master=sw["MASTER"] == "bf16")
        if extras["grad_clip"] > 0 or extras["bf16_master"]:
            use_fused = False                     # both live on the library-collective optimizer path
        if use_fused and rt.device_type == "cuda" and not ops.reference_path():
            from .parallel import symm
            self.comm = symm.create_or_fallback(rt) if rt.world > 1 else symm.SoloComm(rt)
        kind = optimizer_kind or sw["OPT"]
        self.optimizer = setup_optimizer(model, hyper, kind=kind, comm=self.comm, finite_gate=sw["FINITE_GATE"],
                                         overlap_check=sw["OPT_OVERLAP_CHECK"], **extras) if kind == "lean" else \
            setup_optimizer(model, hyper, kind=kind)
        self.tables = None
        if config.table_orders:
            self.tables = HashedTables(config.table_orders, config.table_rows, config.n_embd, seed=config.table_seed, bits=config.table_bits,
                                       device=rt.device, dtype=self.dtype, group=dist.group.WORLD if rt.ddp else None,
                                       world=rt.world, rank=rt.rank, host_state=("auto" if sw["TABLE_HOST_STATE"] == "auto"
                                                   else sw["TABLE_HOST_STATE"].lower() in ("1", "true")),
                                       opt=sw["TABLE_OPT"])
            if self.comm is not None:
                # (row id, gradient) entries this rank records per step and table: one per token
                self.tables.exchange = self.comm.table_exchange(self.tables, self.total_batch // rt.world)
            if init_state is not None:
                self.tables.load_share({k: v for k, v in init_state.items() if k.startswith("table_")})
            model.attach_tables(self.tables)
        self.os1 = None
        if config.os1_rows:
            from .models.os1 import OutputTable
            self.os1 = OutputTable(config, device=rt.device, dtype=self.dtype, group=dist.group.WORLD if rt.ddp else None,
                                   world=rt.world, rank=rt.rank, cap=hyper.os1_cap, eps_rel=hyper.os1_eps_rel)
            model.attach_os1(self.os1)
        if self.comm is not None and config.moe_layers and rt.world > 1:
            self.comm.install_moe(model)
        self.step_index = 0
        self.time_optimizer, self.optimizer_events = False, []
        self.bad_steps = 0
        self.t_start = time.time()
        self._agreed_clock = None                 # set by the step loop once the ranks have exchanged rank 0's clock
        self.sched = dict(lrm=1.0, momentum=hyper.muon_momentum, table_lr=hyper.table_lr)
        self.last_moe_stats = None
        self._dev_x = self._dev_y = None
        self.flops_per_token = model.estimate_flops()

    # ------------------------------------------------------------------------------------------------------
    def set_agreed_clock(self, elapsed_seconds: float) -> None:
        """The training clock every rank agreed on (rank 0's, from the step-control all-reduce).  Everything that is
        decided on the clock -- schedules, the rescue copy, the tail average, the sequence ramp -- reads it through
        ``progress()``, so all ranks cross a threshold on the same step (reference: the MAX-all-reduced
        ``rank0_clock_ms``, round2/source/train.py:22959-22975)."""
        self._agreed_clock = float(elapsed_seconds)

    def progress(self) -> float:
        if self.budget_seconds > 0:
            clock = self._agreed_clock if self._agreed_clock is not None else time.time() - self.t_start
            return min(1.0, clock / self.budget_seconds)
        if self.horizon_steps > 0:
            return min(1.0, self.step_index / self.horizon_steps)
        return 0.0

    def check_device_health(self) -> int:
        """Call where the host synchronises anyway (a forced synchronous step boundary, before a save).  Raises if a
        native kernel gave up on a bounded wait since the last call (training must not go on with data a peer never
        delivered); returns the running count of optimizer steps whose reduced gradient was non-finite (reference:
        ``bad_steps``, round1/source/train.py:10356-10363)."""
        if self.rt.device_type == "cuda" and not ops.reference_path():
            from .ops import _lib
            _lib.check_error_word()
        if self.comm is not None:
            self.comm.check_canaries()           # a write past the end of a peer-mapped buffer
        if hasattr(self.optimizer, "count_bad_steps"):
            self.bad_steps = self.optimizer.count_bad_steps()
        return self.bad_steps

    def h2d(self, inputs: torch.Tensor, targets: torch.Tensor):
        """Host windows -> persistent device tensors (non-blocking from pinned memory)."""
        if self._dev_x is None or self._dev_x.shape != inputs.shape:
            self._dev_x = torch.empty(inputs.shape, dtype=inputs.dtype, device=self.rt.device)
            self._dev_y = torch.empty(targets.shape, dtype=targets.dtype, device=self.rt.device)
        self._dev_x.copy_(inputs, non_blocking=True)
        self._dev_y.copy_(targets, non_blocking=True)
        return self._dev_x, self._dev_y

    def train_step(self, inputs: torch.Tensor, targets: torch.Tensor, micro_steps: int | None = None):
        """One optimizer step on this rank's ``[local_windows, T]`` host (or device) windows."""
        if inputs.device != self.rt.device:
            x_all, y_all = self.h2d(inputs, targets)
        else:
            x_all, y_all = inputs, targets
        accum = micro_steps or self.grad_accum
        if self.config.mtp_offsets:
            sw = switches()
            self.model.set_mtp_weights(schedules.mtp_weights(self.progress(), len(self.config.mtp_offsets),
                                                              sw["MTP_WEIGHT"], sw["MTP_ANNEAL"]))
        db = x_all.shape[0] // self.grad_accum
        opt = self.optimizer
        opt.zero_grad()
        total = None
        for m in range(accum):
            x, y = x_all[m * db:(m + 1) * db], y_all[m * db:(m + 1) * db]
            out = self.model(x, y, loss_div=float(accum))
            if isinstance(out, tuple):
                loss, self.last_moe_stats = out
            else:
                loss = out
            loss.backward()
            opt.accumulate()
            total = loss.detach() if total is None else total + loss.detach()
        self.sched = schedules.apply_schedules(opt, self.hyper, self.step_index, self.progress())
        if self.time_optimizer:          # device time of the step-boundary optimizer chain (events only, read by the caller)
            ev = (torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
            ev[0].record()
            opt.step()
            ev[1].record()
            self.optimizer_events.append(ev)
        else:
            opt.step()
        if "mxfp8" in (self.config.mlp_precision, self.config.attn_proj_precision) and self.rt.device_type == "cuda":
            from .ops import mxfp8
            mxfp8.weights_updated()          # quantised weight copies are refreshed lazily on their next use
        if self.tables is not None:
            self.tables.step(self.sched["table_lr"])
        if self.os1 is not None:
            self.os1.step(x_all.shape[0] // self.grad_accum * accum * x_all.shape[1])
        self.step_index += 1
        return total

    def describe(self) -> str:
        d = self.optimizer.describe() if hasattr(self.optimizer, "describe") else type(self.optimizer).__name__
        return (f"trainer: world {self.rt.world}, dtype {self.dtype}, device_batch {self.device_batch}, grad_accum "
                f"{self.grad_accum}, total_batch {self.total_batch}, flops/token {self.flops_per_token:.3e}; {d}")
