"""The decoder family: dense pre-norm transformer, optional U-net skips, value embeddings, banded attention,
MoE feed-forward blocks and hashed n-gram input tables.

Module and parameter names follow the reference so that its ``model_state`` layout loads unchanged
(round2/source/train.py:11131-11188): ``transformer.wte.weight``, ``transformer.h.{i}.attn.c_q|c_k|c_v|c_proj.weight``,
``transformer.h.{i}.mlp.c_fc|c_proj.weight``, ``transformer.h.{i}.resid_lambda|x0_lambda|ve_lambda``, ``lm_head.weight``,
``value_embeds.{i}.weight``, ``skip_lambda``; MoE blocks: ``mlp.router``, ``mlp.shared.c_fc|c_proj.weight``,
``mlp.w_fc [E,H,d]``, ``mlp.w_proj [E,d,H]``.

Numerics kept from the reference: parameter-free RMSNorm, ``x = a*x + b*x0`` residual mix with ``x0 = norm(embed)``,
rotate-half RoPE followed by QK-RMSNorm, ReLU^2 MLP, untied head padded to a multiple of 64, fp32 logit softcap
``cap*tanh(z/cap)``, cross-entropy with ``ignore_index=-1`` (round2/source/train.py:11612-11709); initialisation
(round2/source/train.py:11233-11278).

Every operator goes through ``them_bones_b200.ops`` which runs the hand-written sm_100a kernels on a GPU and the
plain-PyTorch statement on CPU.
"""
from __future__ import annotations

import math

import torch
import torch.nn as nn

from .. import ops
from ..config import GPTConfig
from ..ref import functional as RF
from .moe import MoeMLP
from .tables import HashedTables


class Linear(nn.Module):
    """Bias-free linear whose weight is ``[out, in]``; the matmul itself is issued by the owning block through
    ``ops`` so that neighbouring weights can be consumed as one fused operand."""

    def __init__(self, n_in: int, n_out: int):
        super().__init__()
        self.weight = nn.Parameter(torch.empty(n_out, n_in))

    def forward(self, x):
        return ops.linear(x, self.weight)


def value_embed_layers(n_layer: int, n_tables: int) -> list:
    """The ``n`` alternating layers that end at the last layer (reference: round2/source/train.py:3299)."""
    return sorted(n_layer - 1 - 2 * j for j in range(n_tables) if n_layer - 1 - 2 * j >= 0)


class CausalSelfAttention(nn.Module):
    def __init__(self, config: GPTConfig, layer: int):
        super().__init__()
        c, a = config.n_embd, config.attn_dim
        self.n_head, self.head_dim = config.n_head, config.head_dim
        self.scale = config.qk_scale if config.qk_scale > 0 else 1.0 / math.sqrt(config.head_dim)
        self.window = config.attn_window if (config.attn_window and layer not in config.attn_long) else 0
        self.precision = config.attn_proj_precision
        self.c_q, self.c_k, self.c_v = Linear(c, a), Linear(c, a), Linear(c, a)
        self.c_proj = Linear(a, c)

    def forward(self, xn, cos, sin, doc_start, ve=None, ve_lambda=None, residual=None):
        b, t, _ = xn.shape
        qkv = ops.linear_qkv(xn, self.c_q.weight, self.c_k.weight, self.c_v.weight, precision=self.precision)
        if ve is not None:
            a = self.n_head * self.head_dim
            qkv = torch.cat([qkv[..., :2 * a], qkv[..., 2 * a:] + ve_lambda.to(qkv.dtype) * ve], dim=-1)
        y = ops.attention(qkv, cos, sin, self.n_head, self.head_dim, self.scale, doc_start, self.window)
        return ops.linear(y, self.c_proj.weight, residual=residual, precision=self.precision)


class MLP(nn.Module):
    def __init__(self, config: GPTConfig):
        super().__init__()
        self.precision = config.mlp_precision
        self.c_fc = Linear(config.n_embd, config.mlp_ratio * config.n_embd)
        self.c_proj = Linear(config.mlp_ratio * config.n_embd, config.n_embd)

    def forward(self, xn, residual=None):
        return ops.mlp(xn, self.c_fc.weight, self.c_proj.weight, residual=residual, precision=self.precision)


class Block(nn.Module):
    def __init__(self, config: GPTConfig, layer: int, has_ve: bool):
        super().__init__()
        # an attention-free block keeps only the MLP; with the "shift1" mixer it first adds a learned multiple of the
        # stream shifted by one token (reference: round1/source/train.py:300-304, 8808-8868)
        has_attn = not config.attn_layers or layer in config.attn_layers
        self.attn = CausalSelfAttention(config, layer) if has_attn else None
        self.mlp = MoeMLP(config, layer) if layer in config.moe_layers else MLP(config)
        self.resid_lambda = nn.Parameter(torch.ones(1))
        self.x0_lambda = nn.Parameter(torch.zeros(1))
        self.ve_lambda = nn.Parameter(torch.zeros(1)) if (has_ve and has_attn) else None
        self.mix_lambda = nn.Parameter(torch.zeros(1)) if (not has_attn and config.mixer == "shift1") else None

    def forward(self, x, x0, cos, sin, doc_start, ve=None, moe_aux=None, x0_acc=None):
        x, xn = ops.resid_mix_norm(x, x0, self.resid_lambda, self.x0_lambda, x0_acc)
        if self.attn is not None:
            x = self.attn(xn, cos, sin, doc_start, ve, self.ve_lambda, residual=x)
            x, xn = ops.norm_split(x)
        elif self.mix_lambda is not None:
            x = x + self.mix_lambda.to(x.dtype) * RF.shift1(x)
            x, xn = ops.norm_split(x)
        if isinstance(self.mlp, MoeMLP):
            return self.mlp(xn, residual=x, moe_aux=moe_aux)
        return self.mlp(xn, residual=x)


class GPT(nn.Module):
    def __init__(self, config: GPTConfig, ep_group=None, ep_world: int = 1, ep_rank: int = 0):
        super().__init__()
        self.config = config
        ve_layers = value_embed_layers(config.n_layer, config.value_embeds)
        self.transformer = nn.ModuleDict(dict(
            wte=nn.Embedding(config.padded_vocab, config.n_embd),
            h=nn.ModuleList([Block(config, i, i in ve_layers) for i in range(config.n_layer)]),
        ))
        self.lm_head = Linear(config.n_embd, config.padded_vocab)
        self.value_embeds = (nn.ModuleDict({str(i): nn.Embedding(config.padded_vocab, config.attn_dim)
                                            for i in ve_layers}) if ve_layers else None)
        self.n_skip = config.n_layer // 2 if config.unet else 0
        self.skip_lambda = nn.Parameter(torch.ones(self.n_skip)) if self.n_skip else None
        self.has_moe = bool(config.moe_layers)
        for blk in self.transformer.h:
            if isinstance(blk.mlp, MoeMLP):
                blk.mlp.set_expert_parallel(ep_group, ep_world, ep_rank)
        self.tables: HashedTables | None = None           # attached by attach_tables(); not nn.Parameters
        self.table_lambda = nn.Parameter(torch.ones(len(config.table_orders))) if config.table_orders else None
        self.os1 = None                                   # output-side table, attached by attach_os1()
        self.answer_weight = None                         # float: the loader marks answer-span targets (target + vocab)
        cos, sin = RF.rotary_tables(config.sequence_len, config.head_dim, config.rope_base)
        self.register_buffer("cos", cos, persistent=False)
        self.register_buffer("sin", sin, persistent=False)

    # ---------------------------------------------------------------------------------------------------------
    @torch.no_grad()
    def init_weights(self, seed: int = 42) -> None:
        cfg = self.config
        nn.init.normal_(self.transformer.wte.weight, mean=0.0, std=0.8)
        nn.init.normal_(self.lm_head.weight, mean=0.0, std=0.001)
        s = math.sqrt(3.0) * cfg.n_embd ** -0.5
        for blk in self.transformer.h:
            if blk.attn is not None:
                for lin in (blk.attn.c_q, blk.attn.c_k, blk.attn.c_v):
                    nn.init.uniform_(lin.weight, -s, s)
                nn.init.zeros_(blk.attn.c_proj.weight)
            if isinstance(blk.mlp, MoeMLP):
                blk.mlp.init_stream(s)
            else:
                nn.init.uniform_(blk.mlp.c_fc.weight, -0.4 * s, 0.4 * s)
                nn.init.zeros_(blk.mlp.c_proj.weight)
            blk.resid_lambda.fill_(1.0)
            blk.x0_lambda.fill_(0.05)
            if blk.ve_lambda is not None:
                blk.ve_lambda.fill_(0.5)
        # extras draw after every base tensor so the base's initial weights do not depend on them
        if self.value_embeds is not None:
            for table in self.value_embeds.values():
                nn.init.normal_(table.weight, mean=0.0, std=0.8)
        if self.skip_lambda is not None:
            self.skip_lambda.fill_(1.0)
        if self.table_lambda is not None:
            self.table_lambda.fill_(1.0)
        for i, blk in enumerate(self.transformer.h):
            if isinstance(blk.mlp, MoeMLP):
                blk.mlp.init_own(s, seed, i)
        cos, sin = RF.rotary_tables(cfg.sequence_len, cfg.head_dim, cfg.rope_base, device=self.cos.device)
        self.cos.copy_(cos)
        self.sin.copy_(sin)

    def cast_compute(self, dtype: torch.dtype):
        """Matrices and tables to the compute dtype; the per-block scalars stay fp32.  cos/sin are rounded to the
        compute dtype like the reference's tables and kept in fp32 storage for the kernels."""
        for name, p in self.named_parameters():
            if p.dim() >= 2:
                p.data = p.data.to(dtype)
        self.cos.copy_(self.cos.to(dtype).float())
        self.sin.copy_(self.sin.to(dtype).float())
        return self

    def attach_tables(self, tables: "HashedTables"):
        self.tables = tables

    def attach_os1(self, table):
        """``models.os1.OutputTable``: its read-out joins the logits before the soft-cap."""
        self.os1 = table

    # ---------------------------------------------------------------------------------------------------------
    def estimate_flops(self) -> float:
        """Training FLOPs per token (forward + backward = 6 x matmul params active per token + attention term;
        reference: round2/source/train.py:11293-11315)."""
        cfg = self.config
        active = 0
        for blk in self.transformer.h:
            if blk.attn is not None:
                active += sum(p.numel() for p in blk.attn.parameters())
            if isinstance(blk.mlp, MoeMLP):
                active += blk.mlp.active_params()
            else:
                active += sum(p.numel() for p in blk.mlp.parameters())
        active += self.lm_head.weight.numel()
        attn = 0
        for blk in self.transformer.h:
            if blk.attn is None:
                continue
            span = min(blk.attn.window or cfg.sequence_len, cfg.sequence_len)
            attn += 12 * cfg.n_head * cfg.head_dim * span / 2       # causal: half the span on average
        return 6 * active + attn

    def num_scaling_params(self) -> int:
        return sum(p.numel() for p in self.parameters())

    def arch_gain_params(self):
        out = []
        if self.skip_lambda is not None:
            out.append(self.skip_lambda)
        if self.table_lambda is not None:
            out.append(self.table_lambda)
        out.extend(blk.ve_lambda for blk in self.transformer.h if blk.ve_lambda is not None)
        out.extend(blk.mix_lambda for blk in self.transformer.h if blk.mix_lambda is not None)
        return out

    # ---------------------------------------------------------------------------------------------------------
    def embed(self, idx, doc_start, table_rows=None):
        x = ops.embedding(idx, self.transformer.wte.weight, self.cos_dtype())
        if self.tables is not None:
            x = self.tables.add_lookup(x, idx, doc_start, self.table_lambda, rows=table_rows)
        return x

    def set_mtp_weights(self, weights) -> None:
        """Per-step weights of the extra targets in ``config.mtp_offsets`` (all zero: next-token loss only)."""
        self.mtp_weights = tuple(float(w) for w in weights)

    def mtp_terms(self, targets, loss_div: float = 1.0):
        """``(targets_k, row_weights_k)`` for every live extra target: position t also predicts the token ``offset``
        places ahead, unless a masked target (document start) lies on the way or the window ends first.  Weights carry
        the schedule weight, the mean over valid next-token targets and ``loss_div`` (reference: ``mtp_terms``,
        round1/source/train.py:5053-5064, there without the document check)."""
        offs, ws = self.config.mtp_offsets, getattr(self, "mtp_weights", ())
        live = [(o, w) for o, w in zip(offs, ws) if w > 0][:2]
        if not live:
            return None
        b, t = targets.shape
        n_valid = (targets >= 0).sum().clamp_min(1).float()
        out = []
        for o, w in live:
            j = o - 1
            tk = torch.full_like(targets, -1)
            tk[:, :t - j] = targets[:, j:]
            ok = tk >= 0
            for s in range(j):                                   # every target between t and t+offset must be real
                ok[:, :t - s] &= targets[:, s:] >= 0
            tk = torch.where(ok, tk, torch.full_like(tk, -1))
            out.append((tk, ok.float() * (w / loss_div) / n_valid))
        return out

    def answer_terms(self, targets, loss_div: float = 1.0):
        """Marked targets (``target + vocab_size``, set by the loader on answer spans) back to targets, and absolute
        row weights ``w / n_valid / loss_div`` with ``w = answer_weight`` where marked and 1 elsewhere: the weighted
        mean over the count of valid targets (reference: ``qa_unmark`` / ``qa_extra_loss``,
        round2/source/train.py:6504-6521)."""
        v = self.config.vocab_size
        marked = targets >= v
        tg = torch.where(marked, targets - v, targets)
        valid = tg >= 0
        w = torch.where(marked, float(self.answer_weight), 1.0) * valid
        return tg, w / valid.sum().clamp_min(1).float() / loss_div

    def cos_dtype(self):
        return self.lm_head.weight.dtype

    def trunk(self, idx, doc_start=None, moe_aux=None, table_rows=None):
        cfg = self.config
        b, t = idx.shape
        if t > self.cos.shape[0]:
            raise ValueError(f"sequence length {t} exceeds the rotary table ({self.cos.shape[0]})")
        if doc_start is None and cfg.doc_mask:
            doc_start = RF.doc_start_positions(idx, cfg.bos_id)
        cos, sin = self.cos[:t], self.sin[:t]
        x = ops.rms_norm(self.embed(idx, doc_start, table_rows))
        x0 = x
        x0_acc = ops.x0_accumulator(x)
        skips = []
        n_layer, n_skip = cfg.n_layer, self.n_skip
        for i, blk in enumerate(self.transformer.h):
            if n_skip and i >= n_layer - n_skip:
                j = i - (n_layer - n_skip)
                x = x + self.skip_lambda[j:j + 1].to(x.dtype) * skips.pop()
            ve = None
            if self.value_embeds is not None and str(i) in self.value_embeds:
                ve = ops.embedding(idx, self.value_embeds[str(i)].weight, x.dtype)
            x = blk(x, x0, cos, sin, doc_start, ve, moe_aux, x0_acc)
            if n_skip and i < n_skip:
                skips.append(x)
        return ops.rms_norm(x)

    def forward(self, idx, targets=None, loss_reduction: str = "mean", loss_div: float = 1.0, doc_start=None,
                row_weights=None, table_rows=None):
        """``targets is None`` -> fp32 softcapped logits ``[B, T, V]``.  Otherwise the loss: ``"mean"`` (scalar,
        divided by ``loss_div``, plus MoE router terms), ``"sum"`` or ``"none"`` (``[B, T]`` per-token nll).  With MoE
        blocks a training forward returns ``(loss, stats)``."""
        cfg = self.config
        moe_aux = [] if (self.has_moe and targets is not None and loss_reduction == "mean") else None
        x = self.trunk(idx, doc_start, moe_aux, table_rows)
        if targets is not None and self.answer_weight is not None:
            targets, aw = self.answer_terms(targets, loss_div)
            if self.training and loss_reduction == "mean" and row_weights is None:
                row_weights = aw
        if self.os1 is not None:
            u, gate = self.os1.read(idx)
            kw = self.os1.readout_args()
            if targets is None:
                return ops.lmhead_logits_os1(x, self.lm_head.weight, cfg.vocab_size, cfg.softcap, u, self.os1.code, gate, **kw)
            if self.training and (cfg.mtp_offsets or cfg.label_smoothing):
                raise ValueError("the output table's loss head has no multi-token or label-smoothing form")
            loss = ops.lmhead_loss_os1(x, self.lm_head.weight, targets, cfg.vocab_size, cfg.softcap, u.view(*idx.shape, -1),
                                       self.os1.code, gate, reduction=loss_reduction, row_weights=row_weights,
                                       loss_div=loss_div, **kw)
        elif targets is None:
            return ops.lmhead_logits(x, self.lm_head.weight, cfg.vocab_size, cfg.softcap)
        else:
            loss = self._plain_loss(x, targets, loss_reduction, loss_div, row_weights)
        if loss_reduction != "mean" or moe_aux is None:
            return loss
        aux = torch.stack([a[0] for a in moe_aux]).sum()
        stats = torch.stack([a[1] for a in moe_aux])
        return loss + aux / loss_div, stats.detach()

    def _plain_loss(self, x, targets, loss_reduction, loss_div, row_weights):
        cfg = self.config
        aux = self.mtp_terms(targets, loss_div) if (loss_reduction == "mean" and self.training) else None
        smooth = cfg.label_smoothing if (self.training and loss_reduction == "mean") else 0.0
        return ops.lmhead_loss(x, self.lm_head.weight, targets, cfg.vocab_size, cfg.softcap,
                               reduction=loss_reduction, row_weights=row_weights, loss_div=loss_div, aux=aux,
                               label_smoothing=smooth)
