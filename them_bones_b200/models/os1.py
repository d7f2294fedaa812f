"""The output-side hashed table: a gradient-trained table read out into the logits.

Role in the model (reference: switch 59, round2/source/train.py:2310-2351; host table ``Os1HostTable`` :3925 and
its worker ``NgramStaleOS1`` :14121-14302): the ``order`` token ids ending at a position are hashed to a row of a
``[rows, dim]`` table and to a pattern of ``dim`` signs; ``u = signs * row`` is scored against a fixed codebook of unit
rows, ``s_v = (u . C_v) / a0``, and the logits receive, before the soft-cap,

    glin * s_v + G_t * beta * relu(sg(s_v) - thr) / (1 - thr)

with ``G_t`` a causal gate computed from the table's own recent reads.  Every row starts at zero, so the first forward
equals the table-free model.  The loss gradient reaches ``u`` through the linear term only; a row's gradient is
``signs * d(u)`` summed over the positions that read it and averaged over the ranks.  The update is the reference's
stateless rule: ``row -= lr g / (rms(g) + eps)``, then the row is scaled back onto ``rms(row) <= cap * lr``.

Where the reference keeps the table in host memory behind a worker thread and exchanges gradients through staging
files, here the rows are sharded over the ranks' HBM (owner = ``row % world``) and travel by the same all-to-all
exchange as the input tables (``parallel.table_a2a``); keys and signs are computed on the device.
"""
from __future__ import annotations

import torch

from .. import ops
from ..ref import functional as RF


class _ReadFn(torch.autograd.Function):
    """Forward: ``u = signs * rows`` for the positions that have a key (zero elsewhere).  Backward: hands
    ``signs * d(u)`` of those positions to the table."""

    @staticmethod
    def forward(ctx, anchor, table, ids, hsign, pos, n_total, dtype):
        ctx.table = table
        ctx.save_for_backward(ids, hsign, pos)
        u = torch.zeros(n_total, table.dim, dtype=dtype, device=ids.device)
        if ids.numel():
            rows = table.exchange.lookup(table.shard, ids, table.world)
            if table.bits and not table.rows_are_views:
                rows = RF.table_view(rows, table.bits)        # straight-through: backward hands d(u) to the master
            u[pos] = ops.os1_apply_signs(rows.to(dtype), hsign)
        return u

    @staticmethod
    def backward(ctx, du):
        ids, hsign, pos = ctx.saved_tensors
        if ids.numel():
            g = ops.os1_apply_signs(du.index_select(0, pos).float(), hsign)
            ctx.table.record_grad(ids, g)
        return torch.zeros(()), None, None, None, None, None, None


class OutputTable:
    def __init__(self, config, *, device="cpu", dtype=torch.float32, group=None, world: int = 1, rank: int = 0,
                 cap: float = 4.0, eps_rel: float = 1e-6, exchange=None):
        rows, dim = config.os1_rows, config.os1_dim
        if rows % world:
            raise ValueError("output-table rows must divide over the ranks")
        self.cfg = config
        self.rows, self.dim, self.order = rows, dim, config.os1_order
        self.world, self.rank, self.group = world, rank, group
        self.device, self.dtype = torch.device(device), dtype
        self.shard = torch.zeros(rows // world, dim, dtype=dtype, device=self.device)
        self.code = RF.os1_codebook(config.padded_vocab, dim, config.os1_code_seed).to(self.device, dtype)
        self.a0 = config.os1_a0 * config.os1_lr
        self.lr, self.cap, self.eps_rel = config.os1_lr, cap, eps_rel
        self.bits, self.rows_are_views = config.os1_bits, False   # 1-bit view (reference: R2_OS1_BITS, :2371-2390)
        self.pending = []
        self._anchor = torch.zeros((), requires_grad=True)
        from ..parallel import table_a2a
        self.exchange = exchange or table_a2a.make_exchange(group, world, rank, self.device)
        self.stats = dict(updates=0, skipped=0, touched=0, capped=0)

    # -- forward --------------------------------------------------------------------------------------------
    def read(self, idx: torch.Tensor):
        """``(u [B*T, dim], gate [B*T])`` for token ids ``[B, T]``; ``u`` carries the table's gradient hook."""
        cfg = self.cfg
        b, t = idx.shape
        row, hs = RF.os1_keys(idx, self.order, self.rows, cfg.bos_id, cfg.os1_seed)
        row, hs = row.reshape(-1), hs.reshape(-1)
        pos = (row >= 0).nonzero().squeeze(1)
        ids, hsel = row.index_select(0, pos), hs.index_select(0, pos)
        if torch.is_grad_enabled():
            u = _ReadFn.apply(self._anchor, self, ids, hsel, pos, b * t, self.dtype)
        else:
            u = _ReadFn.forward(_NoCtx(), None, self, ids, hsel, pos, b * t, self.dtype)
        gate = ops.os1_gate(u.detach(), self.code, idx, self.a0, cfg.os1_gate_w, cfg.os1_gate_h0, cfg.os1_gate_slope)
        return u, gate.reshape(-1)

    def readout_args(self) -> dict:
        cfg = self.cfg
        return dict(a0=self.a0, glin=cfg.os1_glin, beta=cfg.os1_beta, thr=cfg.os1_thr)

    def record_grad(self, ids, g):
        self.pending.append((ids.detach(), g.detach()))

    # -- update ---------------------------------------------------------------------------------------------
    @torch.no_grad()
    def step(self, tokens_per_rank: int):
        """Apply the recorded gradients: route them to the row owners, sum duplicates, average over the ranks, take
        the stateless row step.  ``tokens_per_rank`` (the positions behind the mean loss of this step) sets eps."""
        pend, self.pending = self.pending, []
        if pend:
            ids = torch.cat([p[0] for p in pend])
            grads = torch.cat([p[1] for p in pend]).float()
        else:
            ids = torch.zeros(0, dtype=torch.int64, device=self.device)
            grads = torch.zeros(0, self.dim, device=self.device)
        lids, lgrads = self.exchange.send_grads(ids, grads, self.world)
        ok = torch.isfinite(lgrads).all()
        if self.world > 1:
            ok = self.exchange.all_ok(ok)
        if not bool(ok):
            self.stats["skipped"] += 1
            return
        if lids.numel() == 0:
            return
        uniq, inv = torch.unique(lids, return_inverse=True)
        acc = torch.zeros(len(uniq), self.dim, dtype=torch.float32, device=lgrads.device)
        acc.index_add_(0, inv, lgrads)
        acc /= self.world
        eps = self.eps_rel * RF.os1_typ_rms(self.cfg.os1_glin, self.a0, self.dim, tokens_per_rank, self.world)
        capped = ops.os1_row_step(self.shard, uniq, acc, lr=self.lr, eps=eps, cap=self.cap)
        self.stats["updates"] += 1
        self.stats["touched"] += int(len(uniq))
        self.stats["capped"] += int(capped)

    # -- checkpoint -----------------------------------------------------------------------------------------
    def state_for_checkpoint(self) -> dict:
        """This rank's share as int8 rows with a bf16 row scale (reference: ``os1_table`` / ``os1_scale`` in
        ``model_state``, round2/source/train.py:2339-2341)."""
        t = self.shard.detach().float().cpu()
        if self.bits:
            packed, scale = RF.table_pack_view(t, self.bits)
            return {"os1_table": packed, "os1_scale": scale}
        scale = (t.abs().amax(1, keepdim=True) / 127.0).clamp_min(1e-12).to(torch.bfloat16)
        q = torch.round(t / scale.float()).clamp(-127, 127).to(torch.int8)
        return {"os1_table": q, "os1_scale": scale}

    def load_share(self, state: dict):
        if state["os1_table"].dtype == torch.uint8:
            t = RF.table_unpack_view(state["os1_table"], state["os1_scale"], self.bits)
            self.rows_are_views = True
        else:
            t = state["os1_table"].float() * state["os1_scale"].float()
        if t.shape[0] == self.rows and self.world > 1:
            t = t[self.rank::self.world]
        self.shard.copy_(t.to(self.dtype))


class _NoCtx:
    """Stands in for the autograd context when the read runs without gradients."""

    def save_for_backward(self, *a):
        pass
