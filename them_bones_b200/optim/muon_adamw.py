"""Muon + AdamW optimizer family.

* ``MuonAdamW``       -- single-process reference math (reference: round2/source/train.py:11783-11967).  AdamW groups:
  decoupled decay ``p *= 1 - lr*wd``, ``lerp_`` moments, bias correction.  Muon groups: all matrices of one shape are
  stepped as a stack ``[n, r, c]``: momentum lerp, Nesterov, bf16/fp32 cast, Frobenius normalisation
  ``x / (|x|_F * 1.01 + 1e-6)``, five Polar-Express Newton-Schulz iterations, NorMuon second-moment rescale keeping the
  Frobenius norm, cautious weight decay, ``lr * sqrt(max(1, r/c))``.
* ``DistMuonAdamW``   -- ZeRO-2 style over ``torch.distributed`` (reference: round2/source/train.py:11970-12165): AdamW
  tensors of >= 1024 elements are row-sharded (reduce-scatter AVG, update the slice, all-gather), small ones are
  all-reduced; Muon stacks are padded to a multiple of the world size, reduce-scattered, the owned chunk is
  orthogonalised and all-gathered.  Optimizer state exists only on the owner.
* ``LeanDistMuonAdamW`` (``optim.lean``) -- the production class: low-precision replicas, fp32 masters on owners,
  gradients accumulated straight into the communication buffers, fused in-kernel collectives on NVLink.

``setup_optimizer(model, hyper, ...)`` builds the parameter groups with the reference's split and hyper-parameters
(round2/source/train.py:11498-11577).
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from ..ref import functional as RF


def _is_dist():
    return dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1


class MuonAdamW(torch.optim.Optimizer):
    def __init__(self, param_groups, ns_dtype=None):
        super().__init__(param_groups, defaults={})
        self.ns_dtype = ns_dtype

    def _ns_dtype(self, p):
        if self.ns_dtype is not None:
            return self.ns_dtype
        return torch.bfloat16 if p.is_cuda else torch.float32

    @staticmethod
    def _grad_of(p):
        g = getattr(p, "main_grad", None)
        return g if g is not None else p.grad

    def _adamw_param(self, p, grad, group):
        st = self.state[p]
        if not st:
            st["step"] = 0
            st["exp_avg"] = torch.zeros_like(p, dtype=torch.float32)
            st["exp_avg_sq"] = torch.zeros_like(p, dtype=torch.float32)
            if p.dtype != torch.float32:
                st["master"] = p.detach().float().clone()
        st["step"] += 1
        b1, b2 = group["betas"]
        tgt = st.get("master", p)
        RF.adamw_update(tgt, grad.float(), st["exp_avg"], st["exp_avg_sq"], step=st["step"], lr=group["lr"],
                        beta1=b1, beta2=b2, eps=group["eps"], wd=group["weight_decay"])
        if tgt is not p:
            p.copy_(tgt)

    def _muon_group(self, group):
        params = [p for p in group["params"]]
        if not params:
            return
        p0 = params[0]
        st = self.state[p0]
        n, (r, c) = len(params), p0.shape[-2:]
        lead = p0.shape[:-2]
        if "momentum_buffer" not in st:
            st["momentum_buffer"] = torch.zeros(n, *p0.shape, dtype=torch.float32, device=p0.device)
            sshape = (n, *lead, r, 1) if r >= c else (n, *lead, 1, c)
            st["second_momentum_buffer"] = torch.zeros(sshape, dtype=torch.float32, device=p0.device)
            st["master"] = torch.stack([p.detach().float() for p in params])
        g = torch.stack([(self._grad_of(p).float() if self._grad_of(p) is not None else torch.zeros_like(p, dtype=torch.float32))
                         for p in params])
        if group.get("grad_scale", 1.0) != 1.0:
            g *= group["grad_scale"]
        w = st["master"]
        RF.muon_update(g, w, st["momentum_buffer"], st["second_momentum_buffer"], momentum=group["momentum"],
                       beta2=group["beta2"], lr=group["lr"], wd=group["weight_decay"], ns_steps=group["ns_steps"],
                       ns_dtype=self._ns_dtype(p0))
        for i, p in enumerate(params):
            p.copy_(w[i])

    @torch.no_grad()
    def step(self):
        for group in self.param_groups:
            if group["kind"] == "adamw":
                for p in group["params"]:
                    g = self._grad_of(p)
                    if g is not None:
                        self._adamw_param(p, g, group)
            elif group["kind"] == "muon":
                self._muon_group(group)
            else:
                raise ValueError(f"unknown optimizer kind: {group['kind']}")

    def zero_grad(self, set_to_none: bool = True):
        for group in self.param_groups:
            for p in group["params"]:
                p.grad = None
                mg = getattr(p, "main_grad", None)
                if mg is not None:
                    mg.zero_()

    def accumulate(self):
        """Nothing to fold: autograd accumulates into ``.grad`` (interface parity with the lean class)."""


class DistMuonAdamW(MuonAdamW):
    """Sharded-state variant over ``torch.distributed`` collectives (the NCCL/gloo baseline path)."""

    def __init__(self, param_groups, ns_dtype=None, group=None):
        super().__init__(param_groups, ns_dtype)
        self.group = group
        self.world = dist.get_world_size(group) if _is_dist() else 1
        self.rank = dist.get_rank(group) if _is_dist() else 0

    def _adamw_group_dist(self, group):
        w, r = self.world, self.rank
        for p in group["params"]:
            g = self._grad_of(p)
            if g is None:
                continue
            if p.numel() < 1024 or p.shape[0] % w:
                g32 = g.float()
                dist.all_reduce(g32, op=dist.ReduceOp.SUM, group=self.group)
                self._adamw_param(p, g32 / w, group)
                continue
            rows = p.shape[0] // w
            g32 = g.float().contiguous()
            mine = torch.empty(rows, *p.shape[1:], dtype=torch.float32, device=p.device)
            dist.reduce_scatter_tensor(mine, g32, op=dist.ReduceOp.SUM, group=self.group)
            mine /= w
            st = self.state[p]
            if not st:
                st["step"] = 0
                st["exp_avg"] = torch.zeros_like(mine)
                st["exp_avg_sq"] = torch.zeros_like(mine)
                st["master"] = p.detach()[r * rows:(r + 1) * rows].float().clone()
            st["step"] += 1
            b1, b2 = group["betas"]
            RF.adamw_update(st["master"], mine, st["exp_avg"], st["exp_avg_sq"], step=st["step"], lr=group["lr"],
                            beta1=b1, beta2=b2, eps=group["eps"], wd=group["weight_decay"])
            out = torch.empty_like(p)
            dist.all_gather_into_tensor(out, st["master"].to(p.dtype), group=self.group)
            p.copy_(out)

    def _muon_group_dist(self, group):
        params = group["params"]
        if not params:
            return
        if group.get("moe_local"):
            return self._muon_group(group)          # whole gradient forms locally; no collective
        w, rk = self.world, self.rank
        p0 = params[0]
        n, (r, c) = len(params), p0.shape[-2:]
        k = -(-n // w)
        n_pad = k * w
        st = self.state[p0]
        if "momentum_buffer" not in st:
            st["momentum_buffer"] = torch.zeros(k, r, c, dtype=torch.float32, device=p0.device)
            st["second_momentum_buffer"] = torch.zeros((k, r, 1) if r >= c else (k, 1, c), dtype=torch.float32,
                                                       device=p0.device)
            full = torch.zeros(n_pad, r, c, dtype=torch.float32, device=p0.device)
            for i, p in enumerate(params):
                full[i].copy_(p)
            st["master"] = full[rk * k:(rk + 1) * k].clone()
        slab = torch.zeros(n_pad, r, c, dtype=torch.float32, device=p0.device)
        for i, p in enumerate(params):
            g = self._grad_of(p)
            if g is not None:
                slab[i].copy_(g)
        mine = torch.empty(k, r, c, dtype=torch.float32, device=p0.device)
        dist.reduce_scatter_tensor(mine, slab, op=dist.ReduceOp.SUM, group=self.group)
        mine /= w
        RF.muon_update(mine, st["master"], st["momentum_buffer"], st["second_momentum_buffer"],
                       momentum=group["momentum"], beta2=group["beta2"], lr=group["lr"], wd=group["weight_decay"],
                       ns_steps=group["ns_steps"], ns_dtype=self._ns_dtype(p0))
        out = torch.empty(n_pad, r, c, dtype=p0.dtype, device=p0.device)
        dist.all_gather_into_tensor(out, st["master"].to(p0.dtype), group=self.group)
        for i, p in enumerate(params):
            p.copy_(out[i])

    @torch.no_grad()
    def step(self):
        if self.world == 1:
            return super().step()
        for group in self.param_groups:
            if group.get("moe_local"):
                group["grad_scale"] = 1.0 / self.world     # tokens of every rank reached these experts
                if group["kind"] == "adamw":
                    for p in group["params"]:
                        if self._grad_of(p) is not None:
                            self._adamw_param(p, self._grad_of(p), group)
                else:
                    self._muon_group(group)
            elif group["kind"] == "adamw":
                self._adamw_group_dist(group)
            else:
                self._muon_group_dist(group)


def build_param_groups(model, hyper):
    """The reference's split: embeddings / unembedding / scalars on AdamW, every 2-D hidden matrix on Muon grouped by
    shape, each rank's experts as local groups."""
    from ..models.moe import MoeMLP
    scalar, resid, matrix = [], [], []
    for blk in model.transformer.h:
        resid.append(blk.resid_lambda)
        scalar.append(blk.x0_lambda)
        if blk.attn is not None:
            matrix.extend(blk.attn.parameters())
        matrix.extend(blk.mlp.trunk_parameters() if isinstance(blk.mlp, MoeMLP) else blk.mlp.parameters())
    scalar.extend(model.arch_gain_params())
    emb = list(model.transformer.wte.parameters())
    if model.value_embeds is not None:
        emb.extend(model.value_embeds.parameters())
    head = list(model.lm_head.parameters())
    scale = (model.config.n_embd / 768) ** -0.5
    groups = [
        dict(kind="adamw", name="embed", params=emb, lr=hyper.embedding_lr * scale, betas=(0.8, 0.995), eps=1e-10,
             weight_decay=0.001),
        dict(kind="adamw", name="head", params=head, lr=hyper.unembedding_lr * scale, betas=(0.8, 0.96), eps=1e-10,
             weight_decay=0.01),
        dict(kind="adamw", name="scalars", params=scalar, lr=hyper.scalar_lr, betas=(0.9, 0.95), eps=1e-10,
             weight_decay=0.0),
        dict(kind="adamw", name="resid", params=resid, lr=hyper.scalar_lr / hyper.resid_lr_div, betas=(0.9, 0.95),
             eps=1e-10, weight_decay=0.0),
    ]
    for shape in sorted({tuple(p.shape) for p in matrix}):
        ps = [p for p in matrix if tuple(p.shape) == shape]
        groups.append(dict(kind="muon", name=f"muon{shape}", params=ps, lr=hyper.matrix_lr, momentum=hyper.muon_momentum,
                           beta2=hyper.muon_beta2, ns_steps=hyper.ns_steps, weight_decay=hyper.weight_decay))
    experts = [p for blk in model.transformer.h if isinstance(blk.mlp, MoeMLP) for p in blk.mlp.expert_parameters()]
    for shape in sorted({tuple(p.shape[1:]) for p in experts}):
        ps = [p for p in experts if tuple(p.shape[1:]) == shape]
        groups.append(dict(kind="muon", name=f"experts{shape}", params=ps, lr=hyper.moe_lr,
                           momentum=hyper.muon_momentum, beta2=hyper.muon_beta2, ns_steps=hyper.ns_steps,
                           weight_decay=hyper.weight_decay, moe_local=True))
    for g in groups:
        g["initial_lr"] = g["lr"]
    return groups


def setup_optimizer(model, hyper, kind: str = "auto", group=None, **lean_kw):
    groups = build_param_groups(model, hyper)
    if kind == "auto":
        kind = "lean"
    if kind == "single" or (kind == "dist" and not _is_dist()):
        return MuonAdamW(groups)
    if kind == "dist":
        return DistMuonAdamW(groups, group=group)
    from .lean import LeanDistMuonAdamW
    return LeanDistMuonAdamW(groups, group=group, **lean_kw)
