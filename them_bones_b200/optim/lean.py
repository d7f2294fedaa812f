"""``LeanDistMuonAdamW``: the production optimizer.

What it keeps from the reference's lean class (round2/source/train.py:12253-13411): low-precision replicas with fp32
masters that exist only on the owning rank; gradients accumulated in fp32 *directly in the communication buffers*
(``accumulate()`` after every backward, :12530; every Muon parameter's gradient target is a view of its shape group's
slab, and every parameter itself is a view of the matching weight slab, so publishing updated weights is one gather
into the buffer the model already reads, :13225-13247); one reduce-scatter per slab; row-sharded AdamW tables
(:13136-13148, :13211-13219); all small scalars in one stacked vector reduced by a single all-reduce (:13183-13186);
expert groups stepped locally with gradients scaled by ``1/world`` (:13272-13286); an optional device-side finiteness
gate that zeroes a non-finite step's gradients (:13188-13204); a live cross-check of the fused collectives against the
library ones on the same inputs (``_ovl_check``, :13092-13116).

What is B200-specific: the slabs are allocated from a ``Comm`` object.  ``TorchComm`` uses NCCL/gloo collectives (the
baseline); ``parallel.symm.PeerComm`` places the slabs in NVLink peer-mapped memory and runs the fused kernels: the
reduce-scatter reads every peer's slab chunk by peer loads and feeds the sum straight into the Muon momentum / AdamW
update (no NCCL call, no intermediate buffer), and the updated low-precision shard is stored into every peer's weight
slab by peer stores.
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from ..ref import functional as RF


class TorchComm:
    """Collectives through ``torch.distributed`` (NCCL on GPUs, gloo on CPU)."""

    fused = False

    def __init__(self, group=None):
        self.group = group
        on = dist.is_available() and dist.is_initialized()
        self.world = dist.get_world_size(group) if on else 1
        self.rank = dist.get_rank(group) if on else 0

    def alloc(self, shape, dtype, device):
        return torch.zeros(shape, dtype=dtype, device=device)

    def reduce_scatter_mean(self, full: torch.Tensor, chunk_numel: int) -> torch.Tensor:
        """``full`` is ``[W * chunk]`` flat fp32; returns this rank's averaged chunk (fp32)."""
        if self.world == 1:
            return full.view(-1)[:chunk_numel]
        out = torch.empty(chunk_numel, dtype=full.dtype, device=full.device)
        dist.reduce_scatter_tensor(out, full.view(-1), op=dist.ReduceOp.SUM, group=self.group)
        return out.div_(self.world)

    def all_gather(self, full: torch.Tensor, chunk: torch.Tensor):
        """Publish ``chunk`` (this rank's slice) into every rank's ``full`` (flat ``[W * chunk]``)."""
        if self.world == 1:
            full.view(-1)[:chunk.numel()].copy_(chunk.view(-1))
            return
        dist.all_gather_into_tensor(full.view(-1), chunk.reshape(-1).contiguous(), group=self.group)

    def all_reduce_mean(self, t: torch.Tensor):
        if self.world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.SUM, group=self.group)
            t.div_(self.world)
        return t

    def all_reduce_min(self, t: torch.Tensor):
        if self.world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MIN, group=self.group)
        return t


def plan_muon_counts(shapes, world):
    """How many matrices of each shape group every rank owns.  ``shapes``: ``[(n, rows, cols), ...]`` in group order.
    A group of ``n`` matrices gives every rank ``n // world`` and one more to ``n % world`` ranks; which ranks get the
    extra one is chosen group by group, heaviest groups first, for the ranks with the least Newton-Schulz work so far
    (``max(r, c) * min(r, c)^2`` per matrix), so the step-boundary chain of the busiest rank is as short as the shapes
    allow (reference: ``plan_layout`` / ``ns_flops``, round2/source/train.py:12171-12250).  With a plain
    ``ceil(n / world)`` split of 4 x 20 matrices over 8 ranks, six ranks run 12 orthogonalisations and one runs none;
    here every rank runs 10."""
    cost = [max(r, c) * min(r, c) ** 2 for _, r, c in shapes]
    load = [0.0] * world
    counts = [None] * len(shapes)
    for gi in sorted(range(len(shapes)), key=lambda i: -cost[i]):
        n = shapes[gi][0]
        base, extra = divmod(n, world)
        order = sorted(range(world), key=lambda r: (load[r], r))
        lucky = set(order[:extra])
        counts[gi] = [base + (1 if r in lucky else 0) for r in range(world)]
        for r in range(world):
            load[r] += counts[gi][r] * cost[gi]
    return counts


class _MuonUnit:
    """One shape group: weight slab ``W [n_pad, r, c]`` (replica dtype), gradient slab ``G`` (fp32), owner state for
    ``k = n_pad / world`` slots per rank, of which the first ``counts[rank]`` hold matrices (the rest is padding that the
    fused path skips).  ``slots[i]`` is the slab row of parameter ``i``."""

    def __init__(self, group, params, comm, replica_dtype, master_dtype=torch.float32, counts=None):
        p0 = params[0]
        self.group, self.params = group, params
        self.n, (self.r, self.c) = len(params), p0.shape
        self.k = -(-self.n // comm.world)
        self.n_pad = self.k * comm.world
        if counts is None:
            counts = [min(self.k, max(0, self.n - r * self.k)) for r in range(comm.world)]
        assert sum(counts) == self.n and max(counts) <= self.k
        self.counts, self.kr = list(counts), counts[comm.rank]
        self.slots = [r * self.k + j for r in range(comm.world) for j in range(counts[r])]
        dev = p0.device
        self.W = comm.alloc((self.n_pad, self.r, self.c), replica_dtype, dev)
        self.G = comm.alloc((self.n_pad, self.r, self.c), torch.float32, dev)
        own = slice(comm.rank * self.k, (comm.rank + 1) * self.k)
        full32 = torch.zeros(self.n_pad, self.r, self.c, dtype=torch.float32, device=dev)
        for i, p in enumerate(params):
            full32[self.slots[i]].copy_(p.detach())
        self.master = full32[own].clone().to(master_dtype)     # bf16: updated with stochastic rounding
        self.W.copy_(full32)
        del full32
        for i, p in enumerate(params):
            p.data = self.W[self.slots[i]]
            p.main_grad = self.G[self.slots[i]]
        self.momentum = torch.zeros(self.k, self.r, self.c, dtype=torch.float32, device=dev)
        self.second = torch.zeros((self.k, self.r, 1) if self.r >= self.c else (self.k, 1, self.c),
                                  dtype=torch.float32, device=dev)
        self.own = own


class _RowUnit:
    """One row-sharded AdamW tensor (embedding / head): full replica, fp32 full gradient buffer, owner slice state."""

    def __init__(self, group, p, comm, replica_dtype):
        self.group, self.p = group, p
        dev = p.device
        self.rows = p.shape[0] // comm.world
        self.W = comm.alloc(tuple(p.shape), replica_dtype, dev)
        self.G = comm.alloc(tuple(p.shape), torch.float32, dev)
        self.own = slice(comm.rank * self.rows, (comm.rank + 1) * self.rows)
        self.master = p.detach()[self.own].float().clone()
        self.W.copy_(p.detach())
        p.data = self.W
        p.main_grad = self.G
        self.exp_avg = torch.zeros_like(self.master)
        self.exp_avg_sq = torch.zeros_like(self.master)


class LeanDistMuonAdamW(torch.optim.Optimizer):
    def __init__(self, param_groups, group=None, comm=None, replica_dtype=None, ns_dtype=None, finite_gate=True,
                 overlap_check=False, grad_clip: float = 0.0, bf16_master: bool = False):
        super().__init__(param_groups, defaults={})
        # grad_clip > 0: the reduced gradients are scaled so their global norm does not exceed it (reference: the
        # optional clip of ``GradReducer``, round1/source/train.py:9971-10080).  bf16_master: the Muon matrices' master
        # copies are bf16, written back with stochastic rounding (reference: round1/source/train.py:10219-10226).
        # Both are features of the library-collective path; the fused peer-memory path applies its update inside the
        # reduction kernel and refuses them.
        self.grad_clip, self.bf16_master = float(grad_clip), bool(bf16_master)
        if (self.grad_clip > 0 or self.bf16_master) and getattr(comm, "fused", False):
            raise ValueError("grad_clip / bf16_master need the library-collective optimizer path (BONES_FUSED_COMM=0)")
        self.last_grad_norm = None
        self.comm = comm or TorchComm(group)
        self.world, self.rank = self.comm.world, self.comm.rank
        self.finite_gate = finite_gate
        self.overlap_check = overlap_check
        self.ns_dtype = ns_dtype
        self.replica_dtype = replica_dtype
        self.steps = 0
        self.bad_steps = 0
        self.check_mismatches = 0
        self._build()

    # ------------------------------------------------------------------------------------------------------
    def _build(self):
        comm = self.comm
        self.muon_units, self.row_units, self.local_groups = [], [], []
        small = []                                        # (param, group)
        muon_groups = [g for g in self.param_groups if g["params"] and not g.get("moe_local") and g["kind"] == "muon"]
        plan = plan_muon_counts([(len(g["params"]),) + tuple(g["params"][0].shape) for g in muon_groups], comm.world)
        plan = {id(g): c for g, c in zip(muon_groups, plan)}
        for g in self.param_groups:
            ps = [p for p in g["params"]]
            if not ps:
                continue
            rd = self.replica_dtype or ps[0].dtype
            if g.get("moe_local"):
                self.local_groups.append(g)
            elif g["kind"] == "muon":
                self.muon_units.append(_MuonUnit(g, ps, comm, rd, torch.bfloat16 if self.bf16_master else torch.float32,
                                                 counts=plan[id(g)]))
            else:
                for p in ps:
                    if p.numel() >= 1024 and p.dim() >= 2 and p.shape[0] % comm.world == 0:
                        self.row_units.append(_RowUnit(g, p, comm, self.replica_dtype or p.dtype))
                    else:
                        small.append((p, g))
        # small scalars: one fp32 stack with per-element hyper-parameters
        n = sum(p.numel() for p, _ in small)
        dev = small[0][0].device if small else torch.device("cpu")
        self.S = torch.zeros(n, dtype=torch.float32, device=dev)
        self.SG = comm.alloc((max(n, 1),), torch.float32, dev)[:n]      # peers read it in the fused scalar all-reduce
        self.S_m, self.S_v = torch.zeros_like(self.S), torch.zeros_like(self.S)
        self.small = []
        o = 0
        for p, g in small:
            k = p.numel()
            self.S[o:o + k].copy_(p.detach().reshape(-1))
            p.data = self.S[o:o + k].view(p.shape)
            p.main_grad = self.SG[o:o + k].view(p.shape)
            self.small.append((slice(o, o + k), g))
            o += k
        self._local = MuonLocal(self.local_groups, self.ns_dtype)     # stacks the expert matrices where it can
        if not self._local.stacks:
            for g in self.local_groups:
                for p in g["params"]:
                    p.main_grad = torch.zeros_like(p, dtype=torch.float32)
        self._setup_push()

    def _setup_push(self):
        """Fused GEMM -> reduce-scatter for the Muon matrices: every rank's weight-gradient GEMM adds its tiles straight
        into the gradient slab of the rank that owns the matrix (vector atomics over NVLink from the GEMM epilogue), so
        when backward ends the owner already holds the sum over ranks and nothing is left to reduce at the step boundary.
        Only with the peer-memory communicator on more than one GPU; ``BONES_WGRAD_PUSH=0`` keeps the reduction in the
        optimizer prologue."""
        from ..config import switches
        comm = self.comm
        self.push = bool(getattr(comm, "fused", False) and self.world > 1 and switches()["WGRAD_PUSH"]
                         and hasattr(comm, "peer_addresses"))
        if not self.push:
            return
        for u in self.muon_units:
            addr = comm.peer_addresses(u.G)
            mat = u.r * u.c * 4
            for i, p in enumerate(u.params):
                p.main_grad_push = addr[u.slots[i] // u.k] + u.slots[i] * mat

    def _ns(self, t):
        if self.ns_dtype is not None:
            return self.ns_dtype
        return torch.bfloat16 if t.is_cuda else torch.float32

    @staticmethod
    def _ns_fn(t):
        """The tcgen05 Newton-Schulz on a GPU (unless the plain-PyTorch path is forced), else None."""
        from .. import ops
        if t.is_cuda and not ops.reference_path() and t.shape[-1] % 8 == 0 and t.shape[-2] % 8 == 0:
            from ..ops import muon_native
            return muon_native.newton_schulz
        return None

    # ------------------------------------------------------------------------------------------------------
    @torch.no_grad()
    def accumulate(self):
        """Fold autograd's ``.grad`` into the fp32 communication buffers and drop it.  Kernels that write their weight
        gradient straight into ``main_grad`` leave ``.grad`` unset and nothing is copied for them."""
        for g in self.param_groups:
            for p in g["params"]:
                if p.grad is not None:
                    p.main_grad.add_(p.grad)
                    p.grad = None

    def zero_grad(self, set_to_none: bool = True):
        for u in self.muon_units:
            if not getattr(self, "push", False):          # pushed slabs are cleared by their owner inside step()
                u.G.zero_()
        for u in self.row_units:
            u.G.zero_()
        self.SG.zero_()
        self._local.zero_grad()
        for g in self.param_groups:
            for p in g["params"]:
                p.grad = None

    # ------------------------------------------------------------------------------------------------------
    def _small_vectors(self):
        lr, b1, b2, wd = (torch.empty_like(self.S) for _ in range(4))
        for sl, g in self.small:
            lr[sl], wd[sl] = g["lr"], g["weight_decay"]
            b1[sl], b2[sl] = g["betas"]
        return lr, b1, b2, wd

    @torch.no_grad()
    def step(self):
        comm = self.comm
        self.steps += 1
        if getattr(comm, "fused", False):
            return self._step_fused()
        # 1-3: every reduction first (reference: opt_overlap_rs issues the collectives before any math)
        row_g = [comm.reduce_scatter_mean(u.G, u.master.numel()).view_as(u.master) for u in self.row_units]
        muon_g = [comm.reduce_scatter_mean(u.G, u.momentum.numel()).view_as(u.momentum) for u in self.muon_units]
        comm.all_reduce_mean(self.SG)
        # 4: finiteness gate
        if self.finite_gate:
            sq = self.SG.square().sum()
            for t in row_g + muon_g:
                sq = sq + t.square().sum()
            ok = torch.isfinite(sq).to(torch.float32).reshape(1)
            comm.all_reduce_min(ok)
            okb = ok[0] > 0
            row_g = [torch.where(okb, t, torch.zeros_like(t)) for t in row_g]
            muon_g = [torch.where(okb, t, torch.zeros_like(t)) for t in muon_g]
            self.SG.copy_(torch.where(okb, self.SG, torch.zeros_like(self.SG)))
            self._last_ok = ok
            if not hasattr(self, "_bad_dev"):
                self._bad_dev = torch.zeros(1, dtype=torch.int64, device=ok.device)
            self._bad_dev += (ok <= 0).to(torch.int64)
        # 4b: global-norm clip.  Every rank holds its own shards of the reduced gradients and all of the small ones.
        if self.grad_clip > 0:
            sq = torch.zeros((), dtype=torch.float32, device=self.SG.device)
            for t in row_g + muon_g:
                sq = sq + t.float().square().sum()
            if self.world > 1:
                sq = sq.reshape(1)
                torch.distributed.all_reduce(sq, group=getattr(comm, "group", None))
                sq = sq[0]
            norm = (sq + self.SG.float().square().sum()).sqrt()
            scale = torch.clamp(self.grad_clip / norm.clamp_min(1e-12), max=1.0)
            row_g = [t * scale for t in row_g]
            muon_g = [t * scale for t in muon_g]
            self.SG.mul_(scale)
            self.last_grad_norm = norm
        # 5: updates on the owners' masters
        self._small_step()
        for u, g in zip(self.row_units, row_g):
            b1, b2 = u.group["betas"]
            RF.adamw_update(u.master, g, u.exp_avg, u.exp_avg_sq, step=self.steps, lr=u.group["lr"], beta1=b1,
                            beta2=b2, eps=u.group["eps"], wd=u.group["weight_decay"])
            comm.all_gather(u.W, u.master.to(u.W.dtype))
        for u, g in zip(self.muon_units, muon_g):
            grp = u.group
            master = u.master.float() if self.bf16_master else u.master
            RF.muon_update(g, master, u.momentum, u.second, momentum=grp["momentum"], beta2=grp["beta2"],
                           lr=grp["lr"], wd=grp["weight_decay"], ns_steps=grp["ns_steps"], ns_dtype=self._ns(u.W),
                           ns_fn=self._ns_fn(u.W))
            if self.bf16_master:
                u.master.copy_(RF.stochastic_round_bf16(master))
            comm.all_gather(u.W, u.master.to(u.W.dtype))
        # 5b: local experts
        local_bad = self._local.step(1.0 / self.world)
        if local_bad is not None and self.finite_gate:
            self._bad_dev += local_bad.to(torch.int64) * (self._last_ok > 0).to(torch.int64)   # a step counts once

    def _small_step(self, g=None):
        if not self.small:
            return
        lr, b1, b2, wd = self._small_vectors()
        g = self.SG if g is None else g
        self.S.mul_(1 - lr * wd)
        self.S_m.mul_(b1).add_((1 - b1) * g)
        self.S_v.mul_(b2).add_((1 - b2) * g * g)
        c1, c2 = 1 - b1 ** self.steps, 1 - b2 ** self.steps
        self.S.sub_(lr * (self.S_m / c1) / ((self.S_v / c2).sqrt() + 1e-10))

    def _step_fused(self):
        """In-kernel collectives (``parallel.symm.PeerComm``): one launch per unit reduces the peers' gradient chunks
        over NVLink and applies the owner update; one launch publishes the updated shard into every peer's slab."""
        comm = self.comm
        comm.pre_step()                                   # all ranks' gradients are complete and visible
        sg = comm.all_reduce_mean(self.SG)
        # the matrices and tables are gated element-wise inside their kernels; the scalar stack gets the same gate here,
        # so one non-finite step cannot poison S / S_m / S_v for good
        self._small_step(torch.where(torch.isfinite(sg), sg, torch.zeros_like(sg)))
        for u in self.row_units:
            comm.fused_row_adamw(u, self.steps)
        for u in self.muon_units:
            comm.fused_muon(u, self.steps, self._ns(u.W), own_only=getattr(self, "push", False))
            if getattr(self, "push", False):
                u.G.zero_()                               # consumed; peers add the next step's tiles after post_step()
        local_bad = self._local.step(1.0 / self.world)
        comm.post_step()                                  # every peer's stores into my slabs have landed
        # sum(g^2) of the step, folded into a device-side count of non-finite steps: no host synchronisation in the step
        # and nothing that grows with the number of steps
        if not hasattr(self, "_bad_dev"):
            self._bad_dev = torch.zeros(1, dtype=torch.int64, device=comm.gsq.device)
        bad = ~torch.isfinite(comm.gsq + sg.square().sum())
        if local_bad is not None:
            bad = bad | local_bad
        self._bad_dev += bad.to(torch.int64)
        if self.overlap_check and self.steps == 2:
            self.check_mismatches += comm.cross_check(self)

    # ------------------------------------------------------------------------------------------------------
    def _gather_full(self, full, chunk):
        if self.world == 1:
            full.view(-1)[:chunk.numel()].copy_(chunk.reshape(-1))
        else:
            dist.all_gather_into_tensor(full.view(-1), chunk.reshape(-1).contiguous(),
                                        group=getattr(self.comm, "group", None))

    def consolidated_state_dict(self):
        """Owner masters gathered into full fp32 tensors keyed by parameter (for checkpointing in fp32; reference:
        ``consolidated_state_dict``, round2/source/train.py:13311)."""
        out = {}
        for u in self.muon_units:
            full = torch.empty(u.n_pad, u.r, u.c, dtype=torch.float32, device=u.master.device)
            self._gather_full(full, u.master)
            for i, p in enumerate(u.params):
                out[p] = full[u.slots[i]]
        for u in self.row_units:
            full = torch.empty(u.p.shape, dtype=torch.float32, device=u.master.device)
            self._gather_full(full, u.master)
            out[u.p] = full
        return out

    def unit_state_dict(self) -> dict:
        """This rank's optimizer state (the state lives in the units, not in ``Optimizer.state``): the owner's masters,
        Muon momentum / second moments, AdamW moments, the scalar stack and the local expert state, as host tensors.
        One file per rank restores a run at the same world size; the replicas are rebuilt from the checkpoint's
        ``model_state`` (the consolidated masters) before the optimizer is constructed, so only owner state is kept here
        (the reference never saves optimizer state)."""
        cpu = lambda t: t.detach().cpu().clone()  # noqa: E731
        return {
            "world": self.world, "rank": self.rank, "steps": self.steps,
            "muon": [dict(master=cpu(u.master), momentum=cpu(u.momentum), second=cpu(u.second)) for u in self.muon_units],
            "rows": [dict(master=cpu(u.master), exp_avg=cpu(u.exp_avg), exp_avg_sq=cpu(u.exp_avg_sq)) for u in self.row_units],
            "small": dict(S=cpu(self.S), S_m=cpu(self.S_m), S_v=cpu(self.S_v)),
            "local": [{k: cpu(v) for k, v in self._local.state.get(p, {}).items()}
                      for g in self.local_groups for p in g["params"]],
        }

    @torch.no_grad()
    def load_unit_state_dict(self, sd: dict) -> None:
        if sd["world"] != self.world or sd["rank"] != self.rank:
            raise ValueError(f"optimizer state of rank {sd['rank']}/{sd['world']} loaded on rank {self.rank}/{self.world}")
        self.steps = int(sd["steps"])
        for u, st in zip(self.muon_units, sd["muon"]):
            u.master.copy_(st["master"]); u.momentum.copy_(st["momentum"]); u.second.copy_(st["second"])
        for u, st in zip(self.row_units, sd["rows"]):
            u.master.copy_(st["master"]); u.exp_avg.copy_(st["exp_avg"]); u.exp_avg_sq.copy_(st["exp_avg_sq"])
        self.S.copy_(sd["small"]["S"]); self.S_m.copy_(sd["small"]["S_m"]); self.S_v.copy_(sd["small"]["S_v"])
        ps = [p for g in self.local_groups for p in g["params"]]
        for p, st in zip(ps, sd["local"]):
            if st:
                self._local.load_state(p, st)

    def count_bad_steps(self) -> int:
        """Steps whose reduced gradient held a non-finite value (the fused kernels zeroed those entries).  Synchronises;
        call at a step boundary that synchronises anyway."""
        if hasattr(self, "_bad_dev"):
            self.bad_steps = int(self._bad_dev.item())
        return self.bad_steps

    def describe(self) -> str:
        mu = ", ".join(f"{u.n}x[{u.r},{u.c}] (own {u.kr} of {u.k} slots)" for u in self.muon_units)
        rows = ", ".join(f"[{u.p.shape[0]},{u.p.shape[1]}]/{self.world}" for u in self.row_units)
        return (f"lean optimizer: world {self.world}; muon slabs: {mu}; row tables: {rows}; scalars: {self.S.numel()}; "
                f"local expert groups: {len(self.local_groups)}; comm: {type(self.comm).__name__}")


class _LocalStack:
    """Local expert matrices of one shape as one stack: weights ``W [n, r, c]`` (the parameters become views of it),
    fp32 gradient slab ``G`` (``main_grad`` views), fp32 master, momentum, second moment, and the bf16 Newton-Schulz
    input ``X``.  One reduction-free prologue, one batched Newton-Schulz and one update for all ``n`` matrices."""

    def __init__(self, group, params):
        p0 = params[0]
        self.group, self.params = group, params
        self.r, self.c = p0.shape[-2:]
        counts = [p.numel() // (self.r * self.c) for p in params]
        self.n = n = sum(counts)
        dev = p0.device
        self.W = torch.empty(n, self.r, self.c, dtype=p0.dtype, device=dev)
        self.G = torch.zeros(n, self.r, self.c, dtype=torch.float32, device=dev)
        self.master = torch.empty(n, self.r, self.c, dtype=torch.float32, device=dev)
        self.momentum = torch.zeros_like(self.master)
        self.second = torch.zeros((n, self.r, 1) if self.r >= self.c else (n, 1, self.c), dtype=torch.float32, device=dev)
        self.X = torch.empty(n, self.r, self.c, dtype=torch.bfloat16, device=dev)
        self.sumsq = torch.zeros(n, dtype=torch.float32, device=dev)
        self.views = {}
        o = 0
        for p, e in zip(params, counts):
            sl = slice(o, o + e)
            self.W[sl].copy_(p.detach().reshape(e, self.r, self.c))
            self.master[sl].copy_(p.detach().reshape(e, self.r, self.c))
            p.data = self.W[sl].view(p.shape)
            p.main_grad = self.G[sl].view(p.shape)
            self.views[p] = dict(master=self.master[sl].view(p.shape), momentum=self.momentum[sl].view(p.shape),
                                 second=self.second[sl].view(*p.shape[:-2], *self.second.shape[-2:]))
            o += e


class MuonLocal:
    """Expert groups: the whole gradient forms on this rank; no collective (reference: ``_moe_local_step``)."""

    def __init__(self, groups, ns_dtype=None, native=None):
        """``native``: stack the matrices by shape and step them with the fused prologue / batched tcgen05
        Newton-Schulz / native update kernels (default: when every expert matrix is a bf16 CUDA tensor whose sides are
        multiples of 32 and the plain-PyTorch path is not forced).  Otherwise one PyTorch update per parameter."""
        self.groups, self.ns_dtype, self.state = groups, ns_dtype, {}
        ps = [p for g in groups for p in g["params"]]
        if native is None:
            from .. import ops
            native = bool(ps) and not ops.reference_path() and all(
                p.is_cuda and p.dtype == torch.bfloat16 and p.dim() >= 2 and p.shape[-1] % 32 == 0 and p.shape[-2] % 32 == 0
                for p in ps)
        self.stacks = []
        if native and ps:
            for g in groups:
                by_shape = {}
                for p in g["params"]:
                    by_shape.setdefault(tuple(p.shape[-2:]), []).append(p)
                for plist in by_shape.values():
                    st = _LocalStack(g, plist)
                    self.stacks.append(st)
                    self.state.update(st.views)           # checkpoints read and restore the same tensors
            self.gsq = torch.zeros(1, dtype=torch.float32, device=ps[0].device)

    def zero_grad(self):
        if self.stacks:
            for st in self.stacks:
                st.G.zero_()
        else:
            for g in self.groups:
                for p in g["params"]:
                    p.main_grad.zero_()

    @torch.no_grad()
    def load_state(self, p, st: dict):
        """Restore one parameter's master, momentum and second moment (into the stack's views when stacked)."""
        if p in self.state and self.stacks:
            for k, v in st.items():
                self.state[p][k].copy_(v)
        else:
            self.state[p] = {k: v.to(p.device) for k, v in st.items()}
        p.copy_(self.state[p]["master"])

    @torch.no_grad()
    def _step_stacks(self, grad_scale: float):
        import ctypes
        from ..ops import _lib as L
        from ..ops import muon_native as MN
        _I, _L, _F = ctypes.c_int, ctypes.c_longlong, ctypes.c_float
        self.gsq.zero_()
        for st in self.stacks:
            g = st.group
            mat = st.r * st.c
            n = st.n * mat
            if not hasattr(st, "src"):
                st.src = (ctypes.c_void_p * 1)(ctypes.c_void_p(st.G.data_ptr()))
            st.sumsq.zero_()
            # momentum, Nesterov blend and the per-matrix sum of squares in one pass over the gradient slab (a single
            # source: nothing to reduce); non-finite entries are dropped and show up in gsq
            L.call("bones_rs_muon_prep", st.src, _L(0), _L(n), _I(1), _F(grad_scale), _F(g["momentum"]), L.ptr(st.momentum),
                   L.ptr(st.X), L.ptr(st.sumsq), _L(mat), L.ptr(self.gsq), L.stream())
            L.call("bones_muon_normalize", L.ptr(st.X), L.ptr(st.sumsq), _L(n), _L(mat), L.stream())
            x = MN.newton_schulz(st.X, g["ns_steps"])
            MN.muon_finish(x, st.master, st.second, beta2=g["beta2"], lr=g["lr"], wd=g["weight_decay"])
            st.W.copy_(st.master)
        return ~torch.isfinite(self.gsq)

    @torch.no_grad()
    def step(self, grad_scale: float):
        """Returns a one-element bool tensor, true when any expert gradient of this step was non-finite (None without
        expert groups); no host synchronisation."""
        if self.stacks:
            return self._step_stacks(grad_scale)
        bad = None
        for g in self.groups:
            for p in g["params"]:
                st = self.state.setdefault(p, {})
                r, c = p.shape[-2:]
                if not st:
                    st["master"] = p.detach().float().clone()
                    st["momentum"] = torch.zeros_like(st["master"])
                    st["second"] = torch.zeros((*p.shape[:-2], r, 1) if r >= c else (*p.shape[:-2], 1, c),
                                               dtype=torch.float32, device=p.device)
                grad = p.main_grad * grad_scale
                # per-matrix finiteness gate: an expert whose gradient holds a non-finite value sits the step out
                # (momentum decays, weight decay applies), as the fused kernels do element-wise for the shared matrices
                fin = torch.isfinite(grad).all(dim=-1, keepdim=True).all(dim=-2, keepdim=True)
                grad = torch.where(fin, grad, torch.zeros_like(grad))
                nb = (~fin).any().reshape(1)
                bad = nb if bad is None else bad | nb
                nd = self.ns_dtype or (torch.bfloat16 if p.is_cuda else torch.float32)
                RF.muon_update(grad, st["master"], st["momentum"], st["second"], momentum=g["momentum"],
                               beta2=g["beta2"], lr=g["lr"], wd=g["weight_decay"], ns_steps=g["ns_steps"], ns_dtype=nd,
                               ns_fn=LeanDistMuonAdamW._ns_fn(p))     # the experts' Newton-Schulz on the tcgen05 GEMMs too
                p.copy_(st["master"])
        return bad
