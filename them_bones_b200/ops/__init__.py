"""Operator layer.

Every operator has exactly two bodies: the hand-written sm_100a kernel (``ops.cuda``; autograd ``Function``s around
the native library ``libbones_b200.so``) used whenever the tensors live on a GPU, and the plain-PyTorch statement
(``ref.functional``) used on CPU and when ``BONES_KERNELS=ref`` selects the cuBLAS/SDPA baseline path on a GPU.  A GPU
run whose native library is missing raises instead of silently falling back (reference: a kernel route that does not
apply on the device raises, round2/source/train.py:4964-5042 op registration and its counters ``ATTN_COUNTS``
:4824 / ``MLP_COUNTS`` :6650 that prove a kernel actually fired).

``COUNTS`` records how many times each native body ran.
"""
from __future__ import annotations

import collections
import os

import torch
import torch.nn.functional as F

from ..ref import functional as RF

COUNTS = collections.Counter()
_FORCE_REF = os.environ.get("BONES_KERNELS", "auto") == "ref"


def set_reference_path(flag: bool):
    """True: run the plain-PyTorch bodies even on a GPU (the cuBLAS/SDPA baseline and parity oracle)."""
    global _FORCE_REF
    _FORCE_REF = bool(flag)


def reference_path() -> bool:
    return _FORCE_REF


def native(x: torch.Tensor) -> bool:
    return x.is_cuda and not _FORCE_REF


def _cuda():
    from . import cuda
    return cuda


# --------------------------------------------------------------------------------------------------------------
def embedding(idx, weight, dtype):
    if native(weight):
        return _cuda().embedding(idx, weight, dtype)
    return F.embedding(idx, weight).to(dtype)


def rms_norm(x):
    if native(x):
        return _cuda().rms_norm(x)
    return RF.rms_norm(x)


def norm_split(x):
    """``(x, rms_norm(x))`` for ``x + f(norm(x))``: natively the pass-through gradient is added inside the norm backward."""
    if native(x):
        return _cuda().norm_split(x)
    return x, RF.rms_norm(x)


def x0_accumulator(x):
    """Per-forward accumulator for the gradient of the shared ``x0`` operand of ``resid_mix_norm`` (native path only)."""
    return _cuda().X0Accum() if native(x) and torch.is_grad_enabled() else None


def resid_mix_norm(x, x0, a, b, acc=None):
    """``x' = a*x + b*x0`` and ``rms_norm(x')`` in one pass."""
    if native(x):
        return _cuda().resid_mix_norm(x, x0, a, b, acc)
    xm = RF.resid_mix(x, x0, a, b)
    return xm, RF.rms_norm(xm)


def linear(x, w, residual=None, precision="bf16"):
    """``x @ w.T (+ residual)``; the residual add is fused into the GEMM epilogue on the native path.  ``"mxfp8"``: both
    operands block-quantised along the contraction, in the forward, the input gradient and the weight gradient."""
    if native(x):
        return _cuda().linear(x, w, residual, precision)
    y = _MxLinearRef.apply(x, w.to(x.dtype)) if precision == "mxfp8" else F.linear(x, w.to(x.dtype))
    return y if residual is None else y + residual


def linear_qkv(x, wq, wk, wv, precision="bf16"):
    """Packed ``[.., 3*A]`` projection from three weights.  When the three weights are adjacent rows of one optimizer
    stack the native path reads them as a single ``[3A, C]`` operand with no concatenation."""
    if native(x):
        return _cuda().linear_qkv(x, wq, wk, wv, precision)
    if precision == "mxfp8":
        return torch.cat([_MxLinearRef.apply(x, w.to(x.dtype)) for w in (wq, wk, wv)], dim=-1)
    return torch.cat([F.linear(x, wq.to(x.dtype)), F.linear(x, wk.to(x.dtype)), F.linear(x, wv.to(x.dtype))], dim=-1)


class _MxLinearRef(torch.autograd.Function):
    """Rounding-exact statement of the block-scaled linear: every GEMM sees both operands quantised in 1 x 32 blocks along
    its own contraction axis (reference: the fp8 projections and their fp8 weight gradient,
    round2/source/kernels/nki_attn_tt8g.py:745-757, nki_dw8.py:313-335, there with per-tensor scales)."""

    @staticmethod
    def forward(ctx, x, w):
        ctx.save_for_backward(x, w)
        return (RF.mx_qdq(x.float(), -1) @ RF.mx_qdq(w.float(), -1).T).to(x.dtype)

    @staticmethod
    def backward(ctx, dy):
        x, w = ctx.saved_tensors
        x2, dy2 = x.reshape(-1, x.shape[-1]).float(), dy.reshape(-1, dy.shape[-1]).float()
        dx = RF.mx_qdq(dy2, -1) @ RF.mx_qdq(w.float(), 0)
        dw = RF.mx_qdq(dy2, 0).T @ RF.mx_qdq(x2, 0)
        return dx.view(x.shape).to(x.dtype), dw.to(w.dtype)


def attention(qkv, cos, sin, n_head, head_dim, scale, doc_start=None, window=0):
    if native(qkv):
        return _cuda().attention(qkv, cos, sin, n_head, head_dim, scale, doc_start, window)
    if qkv.is_cuda:
        return _sdpa_attention(qkv, cos, sin, n_head, head_dim, scale, doc_start, window)
    return RF.attention(qkv, cos, sin, n_head, head_dim, scale, doc_start, window)


def _sdpa_attention(qkv, cos, sin, n_head, head_dim, scale, doc_start, window):
    """Baseline GPU path: RoPE and QK-norm as separate torch ops, cuDNN/flash SDPA for the core."""
    b, t, _ = qkv.shape
    c = n_head * head_dim
    q, k, v = qkv.split(c, dim=-1)
    q = RF.rms_norm(RF.apply_rotary(q.reshape(b, t, n_head, head_dim), cos, sin)).transpose(1, 2)
    k = RF.rms_norm(RF.apply_rotary(k.reshape(b, t, n_head, head_dim), cos, sin)).transpose(1, 2)
    v = v.reshape(b, t, n_head, head_dim).transpose(1, 2)
    if doc_start is None and not window:
        y = F.scaled_dot_product_attention(q, k, v, is_causal=True, scale=scale)
    else:
        mask = RF.attention_mask(t, qkv.device, doc_start, window)
        y = F.scaled_dot_product_attention(q, k, v, attn_mask=mask, scale=scale)
    return y.transpose(1, 2).reshape(b, t, c)


def mlp(x, w_fc, w_proj, residual=None, precision="bf16"):
    if native(x):
        return _cuda().mlp(x, w_fc, w_proj, residual, precision)
    if precision == "mxfp8":
        y = _MxMlpRef.apply(x, w_fc.to(x.dtype), w_proj.to(x.dtype))
    else:
        y = RF.mlp(x, w_fc.to(x.dtype), w_proj.to(x.dtype))
    return y if residual is None else y + residual


class _MxMlpRef(torch.autograd.Function):
    """Rounding-exact MXFP8 forward with a straight-through backward whose GEMMs see block-quantised gradients."""

    @staticmethod
    def forward(ctx, x, w_fc, w_proj):
        pre = RF.mx_qdq(x, -1) @ RF.mx_qdq(w_fc, -1).T
        r = F.relu(pre)
        ctx.save_for_backward(x, w_fc, w_proj, r.to(x.dtype))
        return (RF.mx_qdq(r.square(), -1) @ RF.mx_qdq(w_proj, -1).T).to(x.dtype)

    @staticmethod
    def backward(ctx, dy):
        x, w_fc, w_proj, r = ctx.saved_tensors
        shp = x.shape
        x2, dy2, r2 = x.reshape(-1, shp[-1]).float(), dy.reshape(-1, dy.shape[-1]).float(), r.reshape(-1, r.shape[-1]).float()
        dh = RF.mx_qdq(dy2, -1) @ RF.mx_qdq(w_proj.float(), 0)
        dpre = dh * 2.0 * r2
        dx = RF.mx_qdq(dpre, -1) @ RF.mx_qdq(w_fc.float(), 0)
        h = r2.square()
        dw_proj = RF.mx_qdq(dy2, 0).T @ RF.mx_qdq(h, 0)
        dw_fc = RF.mx_qdq(dpre, 0).T @ RF.mx_qdq(x2, 0)
        return dx.view(shp).to(x.dtype), dw_fc.to(w_fc.dtype), dw_proj.to(w_proj.dtype)


def lmhead_logits(x, w, vocab, cap):
    if native(x):
        return _cuda().lmhead_logits(x, w, vocab, cap)
    return RF.softcap_logits(F.linear(x, w.to(x.dtype))[..., :vocab], cap)


def lmhead_loss(x, w, targets, vocab, cap, reduction="mean", row_weights=None, loss_div=1.0, aux=None, label_smoothing=0.0):
    """Loss head: GEMM + softcap + log-sum-exp + target gather in row blocks; the full ``[M, V]`` logits never exist
    on the native path.  ``"mean"`` is divided by ``loss_div`` (gradient accumulation folded into the graph).
    ``row_weights`` (with ``"mean"``): the loss is ``sum(row_weights * nll)`` with absolute weights, nothing else applied.
    ``aux``: up to two ``(targets, row_weights)`` pairs added as ``sum(row_weights * nll(targets))`` -- further targets
    that share each row's soft-max (multi-token prediction; reference: ``fused_loss_multi``,
    round1/source/train.py:5070-5093).  ``label_smoothing``: the main target's loss becomes ``(1 - s) * nll + s * (lse -
    mean_v z_v)`` (reference: the label-smoothing loss-head pair, round2/source/train.py:5697-5767)."""
    if native(x):
        return _cuda().lmhead_loss(x, w, targets, vocab, cap, reduction, row_weights, loss_div, aux, label_smoothing)
    out = RF.softcap_cross_entropy(x, w.to(x.dtype), targets, vocab, cap, row_weights, reduction, label_smoothing)
    # row weights are absolute (they carry the mean and loss_div themselves), as on the native path
    out = out / loss_div if (reduction == "mean" and loss_div != 1.0 and row_weights is None) else out
    if aux and reduction == "mean":
        for tk, wk in aux:
            out = out + RF.softcap_cross_entropy(x, w.to(x.dtype), tk, vocab, cap, wk, "mean")
    return out


# -- output-side hashed table ------------------------------------------------------------------------------------
def os1_apply_signs(x, hsign, out_dtype=None):
    """Rows times their context's sign pattern: ``signs(hsign) * x`` (``x [n, dim]``, ``hsign [n]`` int64)."""
    if native(x):
        return _cuda().os1_apply_signs(x, hsign, out_dtype)
    return (RF.os1_signs(hsign, x.shape[1]) * x.float()).to(out_dtype or x.dtype)


def os1_gate(u, code, idx, a0, width, h0, slope):
    """The read-out's gate ``[B, T]`` (no gradient): see ``ref.functional.os1_gate``.  Native: the per-position dot
    product with the following token's code row is one kernel; the banded mean is a prefix sum."""
    if not native(u):
        return RF.os1_gate(u, code, idx, a0, width, h0, slope)
    with torch.no_grad():
        b, t = idx.shape
        nxt = torch.full((b, t), -1, dtype=torch.int64, device=idx.device)
        nxt[:, :-1] = idx[:, 1:]
        sd = _cuda().os1_gate_dot(u.reshape(b * t, -1), code, nxt.view(-1), a0).view(b, t)
        cs = F.pad(sd.cumsum(1), (1, 0))
        pos = torch.arange(t, device=idx.device)
        lo = (pos - width).clamp_min(0)
        h = (cs[:, pos] - cs[:, lo]) / (pos - lo).clamp_min(1).float()
        return torch.sigmoid(slope * (h - h0))


def lmhead_loss_os1(x, w, targets, vocab, cap, u, code, gate, *, a0, glin, beta, thr, reduction="mean", row_weights=None,
                    loss_div=1.0):
    """Loss head with the output table's term ``glin s + G beta relu(sg(s) - thr) / (1 - thr)``, ``s = u C^T / a0``,
    added to the logits before the soft-cap; the gradient reaches ``u`` through the linear term only."""
    if native(x):
        return _cuda().lmhead_loss_os1(x, w, targets, vocab, cap, u, code, gate, a0, glin, beta, thr, reduction,
                                       row_weights, loss_div)
    out = RF.softcap_cross_entropy_os1(x, w.to(x.dtype), targets, vocab, cap, u, code, gate, a0=a0, glin=glin, beta=beta,
                                       thr=thr, weights=row_weights, reduction=reduction)
    return out / loss_div if (reduction == "mean" and loss_div != 1.0 and row_weights is None) else out


def lmhead_logits_os1(x, w, vocab, cap, u, code, gate, *, a0, glin, beta, thr):
    if native(x):
        return _cuda().lmhead_logits_os1(x, w, vocab, cap, u, code, gate, a0, glin, beta, thr)
    s = F.linear(u.to(x.dtype), code.to(x.dtype)).float()[..., :vocab].reshape(-1, vocab) / a0
    pre = F.linear(x, w.to(x.dtype)).float()[..., :vocab].reshape(-1, vocab) + RF.os1_readout(s, gate.reshape(-1), glin, beta, thr)
    return RF.softcap_logits(pre, cap).view(*x.shape[:-1], vocab)


@torch.no_grad()
def os1_row_step(table, rows, g, *, lr, eps, cap):
    """Stateless row update of the output table, in place on ``table[rows]``; returns how many rows the budget scaled."""
    if native(table):
        return _cuda().os1_row_step(table, rows, g, lr, eps, cap)
    old = table.index_select(0, rows)
    r = g.float().square().mean(1, keepdim=True).sqrt()
    stepped = old.float() - g.float() * (lr / (r + eps))
    new = RF.os1_row_step(old, g, lr, eps, cap)
    table.index_copy_(0, rows, new.to(table.dtype))
    return (stepped.square().mean(1).sqrt() > cap * lr).sum().to(torch.int32).reshape(1)


# -- MoE ---------------------------------------------------------------------------------------------------------
def router_logits(h, router):
    """fp32 router logits ``h @ router^T`` (bf16 inputs, fp32 accumulation)."""
    if native(h):
        return _cuda().router_logits(h, router)
    return F.linear(h.float(), router.float())


def moe_slots(idx, b, t, n_exp, cap):
    """Causal per-sequence capacity slotting: ``(slot [n, k], token_of_slot [E*b*cap])``."""
    if native(idx):
        return _cuda().moe_slots(idx, b, t, n_exp, cap)
    return RF.moe_slots(idx, b, t, n_exp, cap)


def moe_dispatch(h, tok, slot=None):
    """Gather token rows into the slot buffer: ``xs[s] = h[tok[s]]`` and zero where ``tok[s] == n``."""
    if native(h):
        return _cuda().moe_dispatch(h, tok, slot)
    hp = torch.cat([h, h.new_zeros(1, h.shape[1])])
    return hp.index_select(0, tok)


def moe_combine(ys, slot, gates):
    """``out[n] = sum_k gates[n,k] * ys[slot[n,k]]`` with dropped assignments (slot == S) contributing zero."""
    if native(ys):
        return _cuda().moe_combine(ys, slot, gates)
    yp = torch.cat([ys, ys.new_zeros(1, ys.shape[1])])
    out = 0
    for k in range(slot.shape[1]):
        out = out + gates[:, k:k + 1].to(ys.dtype) * yp.index_select(0, slot[:, k])
    return out


def moe_dispatch_exchange(h, tok, group, world, n_exp, slot=None, key=None):
    from ..parallel import moe_a2a
    return moe_a2a.dispatch_exchange(h, tok, group, world, n_exp, slot, key)


def moe_exchange(xs, group, world, n_exp, forward=True, key=None):
    from ..parallel import moe_a2a
    return moe_a2a.exchange(xs, group, world, n_exp, forward, key)


def moe_experts(xs, w_fc, w_proj, precision="bf16"):
    """Local experts on rows grouped ``[E_local, rows_per_expert, d]``."""
    e = w_fc.shape[0]
    if native(xs):
        return _cuda().moe_experts(xs, w_fc, w_proj, precision)
    x3 = xs.view(e, -1, xs.shape[-1])
    if precision == "mxfp8":
        return torch.cat([_MxMlpRef.apply(x3[j], w_fc[j].to(xs.dtype), w_proj[j].to(xs.dtype)) for j in range(e)])
    h = RF.relu2(torch.bmm(x3, w_fc.to(xs.dtype).transpose(1, 2)))
    return torch.bmm(h, w_proj.to(xs.dtype).transpose(1, 2)).reshape(xs.shape)


# -- tables ------------------------------------------------------------------------------------------------------
@torch.no_grad()
def sparse_adam_rows(table, rows, g, m, v, *, step, lr, beta1, beta2, eps, decay):
    """Adam on the touched rows only (in place on ``table[rows]``, ``m``, ``v``)."""
    if native(table):
        return _cuda().sparse_adam_rows(table, rows, g, m, v, step, lr, beta1, beta2, eps, decay)
    m.lerp_(g, 1 - beta1)
    v.lerp_(g.square(), 1 - beta2)
    b1, b2 = 1 - beta1 ** step, 1 - beta2 ** step
    w = table.index_select(0, rows).float()
    w = w * (1 - lr * decay) - lr * (m / b1) / ((v / b2).sqrt() + eps)
    table.index_copy_(0, rows, w.to(table.dtype))
