"""Expert-parallel mixture-of-experts feed-forward block.

Semantics follow the reference's MoE (round2/source/train.py:10463-11067): an fp32 router, softmax, top-k (k=1: the
probability is the gate; k=2: gates renormalised over the two), a *causal per-sequence* capacity ``C`` counted left to
right so that a token's routing never depends on later tokens, a slot buffer laid out ``[E, b, C]`` whose expert-e chunk
travels to the rank that holds expert e, a ReLU^2 expert MLP, the mirror exchange, a gate-weighted combine, an optional
always-on shared MLP half, and the Switch load-balance + z-loss router terms.  The reference requires
``experts == world``; here ``E = m * W`` experts are sharded ``m`` per rank.

Experts are drawn from per-expert generators seeded by (run seed, layer, expert) so every rank layout builds identical
experts (reference: ``moe_seed``, round2/source/train.py:10499-10502).
"""
from __future__ import annotations

import hashlib

import torch
import torch.nn as nn
import torch.nn.functional as F

from .. import ops
from ..config import GPTConfig
from ..ref import functional as RF


def moe_seed(*parts) -> int:
    return int(hashlib.md5(":".join(str(p) for p in ("moe",) + parts).encode("ascii")).hexdigest()[:15], 16)


class SharedMLP(nn.Module):
    def __init__(self, n_embd: int, hidden: int):
        super().__init__()
        from .gpt import Linear
        self.c_fc = Linear(n_embd, hidden)
        self.c_proj = Linear(hidden, n_embd)


class MoeMLP(nn.Module):
    def __init__(self, config: GPTConfig, layer: int):
        super().__init__()
        self.layer = layer
        self.n_exp, self.topk, self.cap = config.moe_experts, config.moe_topk, config.moe_capacity
        self.hidden, self.n_embd = config.moe_hidden, config.n_embd
        self.aux_w, self.z_w = config.moe_aux, config.moe_zloss
        self.precision = config.mlp_precision
        self.router = nn.Parameter(torch.zeros(self.n_exp, config.n_embd))
        self.shared = SharedMLP(config.n_embd, config.moe_shared) if config.moe_shared else None
        self.ep_group, self.ep_world, self.ep_rank = None, 1, 0
        self.w_fc = nn.Parameter(torch.empty(self.n_exp, self.hidden, config.n_embd))
        self.w_proj = nn.Parameter(torch.empty(self.n_exp, config.n_embd, self.hidden))
        self.w_fc.moe_local = True
        self.w_proj.moe_local = True
        self.last_stats = None

    # -- layout ---------------------------------------------------------------------------------------------
    def set_expert_parallel(self, group, world: int, rank: int):
        """Keep only this rank's ``E / world`` experts (expert e lives on rank ``e // (E / world)``)."""
        if self.n_exp % world:
            raise ValueError(f"{self.n_exp} experts do not divide over {world} expert-parallel ranks")
        self.ep_group, self.ep_world, self.ep_rank = group, world, rank
        if world > 1:
            m = self.n_exp // world
            for name in ("w_fc", "w_proj"):
                old = getattr(self, name)
                new = nn.Parameter(old.data[rank * m:(rank + 1) * m].clone())
                new.moe_local = True
                setattr(self, name, new)

    @property
    def local_experts(self) -> int:
        return self.n_exp // self.ep_world

    def trunk_parameters(self):
        out = [self.router]
        if self.shared is not None:
            out += [self.shared.c_fc.weight, self.shared.c_proj.weight]
        return out

    def expert_parameters(self):
        return [self.w_fc, self.w_proj]

    def active_params(self) -> int:
        n = self.router.numel() + self.topk * 2 * self.hidden * self.n_embd
        if self.shared is not None:
            n += sum(p.numel() for p in self.shared.parameters())
        return n

    # -- init -----------------------------------------------------------------------------------------------
    @torch.no_grad()
    def init_stream(self, s: float):
        """Draws taken from the model's main random stream (the shared half, as a dense MLP would)."""
        if self.shared is not None:
            nn.init.uniform_(self.shared.c_fc.weight, -0.4 * s, 0.4 * s)
            nn.init.zeros_(self.shared.c_proj.weight)

    @torch.no_grad()
    def init_own(self, s: float, seed: int, layer: int):
        g = torch.Generator().manual_seed(moe_seed(seed, layer, "router"))
        self.router.copy_(torch.empty(self.router.shape).uniform_(-s, s, generator=g))
        m = self.local_experts
        for j in range(m):
            e = self.ep_rank * m + j
            g = torch.Generator().manual_seed(moe_seed(seed, layer, e))
            self.w_fc[j].copy_(torch.empty(self.hidden, self.n_embd).uniform_(-0.4 * s, 0.4 * s, generator=g))
            self.w_proj[j].zero_()

    # -- forward --------------------------------------------------------------------------------------------
    def forward(self, xn, residual=None, moe_aux=None):
        b, t, d = xn.shape
        n = b * t
        h = xn.reshape(n, d)
        logits = ops.router_logits(h, self.router)
        p, idx, gates = RF.moe_route(logits, self.topk)
        # a sequence of t tokens cannot send more than t of them to one expert: the same routing with a smaller slot
        # buffer for short inputs (a decode step is one token per sequence)
        cap = min(self.cap, t)
        slot, tok = ops.moe_slots(idx, b, t, self.n_exp, cap)
        # slot gather ([E*b*C, d], empty slots are zero rows) + exchange to the expert owners
        xs = ops.moe_dispatch_exchange(h, tok, self.ep_group, self.ep_world, self.n_exp, slot, key=self.layer)
        ys = ops.moe_experts(xs, self.w_fc, self.w_proj, self.precision)   # rows grouped by local expert
        ys = ops.moe_exchange(ys, self.ep_group, self.ep_world, self.n_exp, forward=False, key=self.layer)
        out = ops.moe_combine(ys, slot, gates)                            # [n, d]
        if self.shared is not None:
            out = out + ops.mlp(h, self.shared.c_fc.weight, self.shared.c_proj.weight, precision=self.precision)
        out = out.view(b, t, d)
        if residual is not None:
            out = out + residual
        if moe_aux is not None:
            aux, lb, z, f = RF.moe_aux_terms(p, logits, idx, self.n_exp, self.topk, self.aux_w, self.z_w)
            kept = (slot < self.n_exp * b * cap).float().mean()
            moe_aux.append((aux, torch.cat([torch.stack([kept, lb.detach(), z.detach()]), f.detach()])))
        return out
