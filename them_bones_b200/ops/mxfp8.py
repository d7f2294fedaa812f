"""MXFP8 (OCP microscaling, E4M3 elements, UE8M0 scale per 1 x 32 block) operators on the CTA-pair block-scaled GEMM
(``csrc/gemm_mxfp8_2cta.cu``).

``mlp`` is the fused ReLU^2 MLP, ``_MxLinearFn`` the block-scaled projection (attention qkv / out), ``_MxExpertsFn`` the
grouped experts.  In each of them the forward GEMM, the input-gradient GEMM and the weight-gradient GEMM all run in
MXFP8: activations and gradients are quantised along the axis the consuming GEMM contracts over -- by the producing
GEMM's epilogue where there is one, else by one pass of the dual-axis quantiser -- and the weight gradients accumulate in
fp32 straight into the optimizer's slab.

Weights are quantised once per optimizer step, in both orientations (along ``in`` for forward, along ``out`` for dX), and
cached until ``weights_updated()`` is called (reference: the per-step fp8 scale / pre-cast refresh,
``fp8_refresh_weights`` round2/source/train.py:6617-6657, and its per-step quantised-weight caches keyed on an epoch,
round1/source/train.py:2059-2076).
"""
from __future__ import annotations

import ctypes
import os

import torch

from . import COUNTS
from . import _lib as L
from . import cuda as C

_I, _L, _F = ctypes.c_int, ctypes.c_longlong, ctypes.c_float
_EPOCH = [0]
_CACHE = {}


def weights_updated():
    """Invalidate every cached quantised weight (call after each optimizer step)."""
    _EPOCH[0] += 1


GE_BF16, GE_BF16_RES, GE_RELU2, GE_ACC_F32, GE_MUL_2SQRT = 0, 1, 2, 3, 4
# Tile N of forward / input-gradient GEMMs.  224 keeps two accumulators in TMEM, so a tile's epilogue hides behind the
# next tile's MMAs: the choice for a short contraction or a quantising epilogue.  256 (one accumulator) moves fewer
# operand bytes per flop and wins once the contraction is long enough to dwarf the exposed epilogue (measured on
# 65536 x 1280 x 5120: 2316 against 2212 TFLOP/s).  BONES_MX_BN=160|224|256 forces one value.
_BN_FORCED = int(os.environ.get("BONES_MX_BN", 0))
BN_FWD = _BN_FORCED or 224
BN_WGRAD = 256                                             # weight gradients: MN-major operands, one accumulator


def bn_for(k: int, heavy_epilogue: bool = False) -> int:
    if _BN_FORCED:
        return _BN_FORCED
    return 256 if (k >= 2560 and not heavy_epilogue) else 224


def sf2_bytes(rows: int, k: int, group: int = 128) -> int:
    return -(-rows // group) * -(-k // 128) * -(-group // 128) * 512


def _sf_buf(rows: int, k: int, group: int, dev, lead=()):
    """Scale-chunk buffer of an operand.  When the rows fill whole tiles of whole 128-row chunks and K whole 128-blocks
    every byte is written by the producing kernel; otherwise the slots of rows that do not exist must read as zero."""
    full = group % 128 == 0 and rows % group == 0 and k % 128 == 0
    mk = torch.empty if full else torch.zeros
    return mk(*lead, sf2_bytes(rows, k, group), dtype=torch.uint8, device=dev)


def quant2(x2: torch.Tensor, *, row: bool = True, col: bool = False, group_r: int = 128, group_c: int = 128, out=None):
    """bf16 ``[R, C]`` -> ``(q_row, sf_row, q_col, sf_col)``: E4M3 copies quantised in 1 x 32 blocks along C (``row``) and
    along R (``col``), each with UE8M0 scale chunks laid out for an operand whose tiles are ``group`` rows.  The column
    copy's chunks describe the transposed operand (rows = C, contraction = R) that a weight-gradient GEMM reads.
    ``out``: the same four tensors preallocated (slices of a batch)."""
    r, c = x2.shape
    dev = x2.device
    qr = sfr = qc = sfc = None
    if out is not None:
        qr, sfr, qc, sfc = out
    else:
        if row:
            qr = torch.empty(r, c, dtype=torch.uint8, device=dev)
            sfr = _sf_buf(r, c, group_r, dev)
        if col:
            qc = torch.empty(r, c, dtype=torch.uint8, device=dev)
            sfc = _sf_buf(c, r, group_c, dev)
    L.call("bones_mx2_quant", L.ptr(x2), _L(x2.stride(0)), L.ptr(qr), L.ptr(sfr), _I(group_r), L.ptr(qc), L.ptr(sfc), _I(group_c),
           _L(r), _L(c), L.stream())
    COUNTS["mx_quant"] += 1
    return qr, sfr, qc, sfc


def weight_q2_batched(w3: torch.Tensor, transposed: bool, bn: int):
    """Per-expert quantised weights ``[E, out, in]`` -> ``(q [E, rows, k], sf [E, bytes])`` (``transposed``: of ``w^T``)."""
    key = (w3.data_ptr(), tuple(w3.shape), transposed, bn, "b")
    ent = _CACHE.get(key)
    if ent is None or ent[0] != _EPOCH[0] or ent[1] != w3._version:
        src = w3.detach().transpose(1, 2).contiguous() if transposed else w3.detach()
        e, rows, k = src.shape
        q = torch.empty(e, rows, k, dtype=torch.uint8, device=w3.device)
        sf = torch.zeros(e, sf2_bytes(rows, k, bn), dtype=torch.uint8, device=w3.device)
        for j in range(e):
            quant2(src[j], group_r=bn, out=(q[j], sf[j], None, None))
        ent = (_EPOCH[0], w3._version, q, sf)
        _CACHE[key] = ent
    return ent[2], ent[3]


def weight_q2(w: torch.Tensor, transposed: bool, bn: int):
    """Quantised weight as the B operand of a GEMM with tile N ``bn``: ``x @ w.T`` (``transposed=False``: blocks along
    ``in``) or ``dy @ w`` (``True``: ``w.T``, blocks along ``out``).  Cached until ``weights_updated()``."""
    key = (w.data_ptr(), tuple(w.shape), transposed, bn)
    ent = _CACHE.get(key)
    if ent is None or ent[0] != _EPOCH[0] or ent[1] != w._version:
        src = w.detach().t().contiguous() if transposed else w.detach()
        q, sf, _, _ = quant2(src, group_r=bn)
        ent = (_EPOCH[0], w._version, q, sf)
        _CACHE[key] = ent
    return ent[2], ent[3]


def gemm2(aq, sfa, bq, sfb, m, n, k, *, a_major=0, b_major=0, epi=GE_BF16, r=None, alpha=1.0, beta=1.0, bn=None, out=None,
          want_d=True, want_q=False, want_t=False, dq_group=128, dt_group=128, splits=0, batch=1):
    """``epilogue(alpha * A B^T)`` on the CTA-pair block-scaled kernel.  ``aq``: ``[m, k]`` (``a_major=0``) or ``[k, m]``
    (``a_major=1``) E4M3; ``bq`` likewise with ``n``.  ``batch > 1``: every operand carries a leading batch axis and is
    contiguous (grouped experts).  Returns ``(d, dq, dsf, dt, dtsf)``: the bf16 result (``out`` for the fp32 accumulate
    form), its copy quantised along ``n`` and its copy quantised along ``m`` (None where not asked)."""
    bn = bn or (BN_WGRAD if b_major else BN_FWD)
    dev = aq.device
    lead = (batch,) if batch > 1 else ()
    d = out
    if d is None and want_d:
        d = torch.empty(*lead, m, n, dtype=torch.float32 if epi == GE_ACC_F32 else torch.bfloat16, device=dev)
    dq = dsf = dt = dtsf = None
    if want_q:
        dq = torch.empty(*lead, m, n, dtype=torch.uint8, device=dev)
        dsf = _sf_buf(m, n, dq_group, dev, lead)
    if want_t:
        dt = torch.empty(*lead, m, n, dtype=torch.uint8, device=dev)
        dtsf = _sf_buf(n, m, dt_group, dev, lead)
    sa, sb = (aq.stride(0), bq.stride(0)) if batch > 1 else (0, 0)
    lda, ldb = aq.stride(-2), bq.stride(-2)
    sd = d.stride(0) if (d is not None and batch > 1) else 0
    ldd = d.stride(-2) if d is not None else 0
    sr = r.stride(0) if (r is not None and batch > 1) else 0
    ldr = r.stride(-2) if r is not None else 0
    L.call("bones_gemm_mxfp8_pair", L.ptr(aq), L.ptr(sfa), L.ptr(bq), L.ptr(sfb), L.ptr(d), L.ptr(r), L.ptr(dq), L.ptr(dsf),
           _I(dq_group), L.ptr(dt), L.ptr(dtsf), _I(dt_group), _I(m), _I(n), _I(k), _I(batch), _L(lda), _L(ldb), _L(ldd), _L(ldr),
           _L(sa), _L(sb), _L(sd), _L(sr), _I(a_major), _I(b_major), _I(epi), _F(alpha), _F(beta), _I(bn), _I(splits), _I(0),
           L.stream())
    COUNTS["mx_gemm"] += 1
    return d, dq, dsf, dt, dtsf


def wgrad2_into(dyq_c, dysf_c, xq_c, xsf_c, grad32, col0: int = 0, n_out: int | None = None):
    """``grad32 [n_out, in] += dY[:, col0:col0+n_out]^T X``: the rows ``col0 ..`` of the output channels (a multiple of 128,
    so their scale chunks are a contiguous run) of a token-axis-quantised ``dY``."""
    tokens, total = dyq_c.shape
    n_out = total if n_out is None else n_out
    kb = -(-tokens // 128)
    a = dyq_c[:, col0:col0 + n_out]
    sfa = dysf_c[(col0 // 128) * kb * 512:]
    gemm2(a, sfa, xq_c, xsf_c, n_out, xq_c.shape[1], tokens, a_major=1, b_major=1, epi=GE_ACC_F32, out=grad32, bn=BN_WGRAD)


def wgrad2(dyq_c, dysf_c, xq_c, xsf_c, w):
    """``dW[out, in] += dY^T X`` with both activations quantised along the token axis (MN-major operands), accumulated in
    fp32 straight into the weight's gradient slab (reference: the fp8 weight-gradient GEMM,
    round2/source/kernels/nki_dw8.py:239, routed by ``dw8_grad`` round2/source/train.py:8185)."""
    tokens, n_out = dyq_c.shape
    n_in = xq_c.shape[1]
    g = getattr(w, "main_grad", None)
    ret = None
    if g is None:
        g = ret = torch.zeros(n_out, n_in, dtype=torch.float32, device=dyq_c.device)
    gemm2(dyq_c, dysf_c, xq_c, xsf_c, n_out, n_in, tokens, a_major=1, b_major=1, epi=GE_ACC_F32, out=g, bn=BN_WGRAD)
    return ret.to(w.dtype) if ret is not None else None


def linear2(x2: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    xq, xsf, _, _ = quant2(x2)
    bn = bn_for(x2.shape[1])
    wq, wsf = weight_q2(w, False, bn)
    return gemm2(xq, xsf, wq, wsf, x2.shape[0], w.shape[0], x2.shape[1], bn=bn)[0]


class _MxLinearFn(torch.autograd.Function):
    """``x @ W^T (+ residual)`` for one weight or several row-adjacent ones (q, k, v), all three GEMMs block-scaled:
    forward ``x_row W_row^T``, input gradient ``dy_row (W^T)_row^T``, weight gradient ``dy_col^T x_col`` accumulated in fp32
    straight into the optimizer's gradient slab (reference: ``AttnProj8PC`` round2/source/train.py:7812 and
    ``attn8_weight_grad`` :8231)."""

    @staticmethod
    def forward(ctx, x, residual, *ws):
        shp = x.shape
        x2 = C._c(x).view(-1, shp[-1])
        m, c = x2.shape
        pad = -m % 128
        if pad:
            x2 = torch.nn.functional.pad(x2, (0, 0, 0, pad))
        w = C._fused_rows(ws) if len(ws) > 1 else ws[0]
        if w is None:
            w = torch.cat(ws, 0)
        n = w.shape[0]
        xq, xsf, xq_c, xsf_c = quant2(x2, col=True, group_c=BN_WGRAD)
        bn = bn_for(c)
        wq, wsf = weight_q2(w, False, bn)
        r2 = None
        if residual is not None:
            r2 = C._c(residual).view(-1, n)
            if pad:
                r2 = torch.nn.functional.pad(r2, (0, 0, 0, pad))
        y = gemm2(xq, xsf, wq, wsf, m + pad, n, c, epi=GE_BF16_RES if r2 is not None else GE_BF16, r=r2, bn=bn)[0]
        ctx.save_for_backward(xq_c, xsf_c, w)
        ctx.ws, ctx.has_res, ctx.shp, ctx.m = ws, residual is not None, shp, m
        COUNTS["linear_mxfp8"] += 1
        return y[:m].view(*shp[:-1], n)

    @staticmethod
    def backward(ctx, dy):
        xq_c, xsf_c, w = ctx.saved_tensors
        mp, c = xq_c.shape
        n, m = w.shape[0], ctx.m
        dy2 = C._c(dy).view(m, n)
        if mp != m:
            dy2 = torch.nn.functional.pad(dy2, (0, 0, 0, mp - m))
        dyq, dysf, dyq_c, dysf_c = quant2(dy2, row=ctx.needs_input_grad[0], col=True, group_c=128)
        dx = None
        if ctx.needs_input_grad[0]:
            bn = bn_for(n)
            wtq, wtsf = weight_q2(w, True, bn)
            dx = gemm2(dyq, dysf, wtq, wtsf, mp, c, n, bn=bn)[0][:m].view(ctx.shp)
        ws = ctx.ws
        grads = [getattr(wi, "main_grad", None) for wi in ws]
        outs = []
        if all(g is not None for g in grads):
            fused = C._fused_rows(grads) if len(grads) > 1 else grads[0]
            if fused is not None:
                wgrad2_into(dyq_c, dysf_c, xq_c, xsf_c, fused)
            else:
                o = 0
                for wi, g in zip(ws, grads):
                    wgrad2_into(dyq_c, dysf_c, xq_c, xsf_c, g, o, wi.shape[0])
                    o += wi.shape[0]
            outs = [None] * len(ws)
        else:
            full = torch.zeros(n, c, dtype=torch.float32, device=dy.device)
            wgrad2_into(dyq_c, dysf_c, xq_c, xsf_c, full)
            o = 0
            for wi in ws:
                outs.append(full[o:o + wi.shape[0]].to(wi.dtype))
                o += wi.shape[0]
        return (dx, dy if ctx.has_res else None) + tuple(outs)


def applies(x, w_fc, w_proj) -> bool:
    c, f = w_fc.shape[1], w_fc.shape[0]
    return x.dtype == torch.bfloat16 and c % 128 == 0 and f % 128 == 0


class _MxMlpFn(torch.autograd.Function):
    """Six block-scaled GEMMs and two quantiser passes per layer.  Forward: ``x`` is quantised once along both axes; the
    c_fc epilogue applies ReLU^2 and emits ``h`` in bf16 (kept for the ReLU^2 backward) and in MXFP8 along the hidden axis
    (c_proj's operand) and along the token axis (kept for ``dW_proj``).  Backward: ``dy`` is quantised along both axes;
    ``dpre = (dy W_proj) * 2 sqrt(h)`` leaves its GEMM only in MXFP8, along the hidden axis for ``dx = dpre W_fc`` and along
    the token axis for ``dW_fc``; both weight gradients are block-scaled GEMMs over the token axis."""

    @staticmethod
    def forward(ctx, x, w_fc, w_proj, residual):
        shp = x.shape
        x2 = C._c(x).view(-1, shp[-1])
        m, c = x2.shape
        f = w_fc.shape[0]
        pad = -m % 128
        if pad:                                    # the token axis is a contraction axis in backward: whole K blocks
            x2 = torch.nn.functional.pad(x2, (0, 0, 0, pad))
        mp = m + pad
        xq, xsf, xq_c, xsf_c = quant2(x2, col=True, group_c=BN_WGRAD)
        bn1, bn2 = bn_for(c, True), bn_for(f)
        wq, wsf = weight_q2(w_fc, False, bn1)
        h, hq, hsf, hq_c, hsf_c = gemm2(xq, xsf, wq, wsf, mp, f, c, epi=GE_RELU2, want_q=True, want_t=True, dt_group=BN_WGRAD,
                                        bn=bn1)
        pq, psf = weight_q2(w_proj, False, bn2)
        r2 = None
        if residual is not None:
            r2 = C._c(residual).view(-1, w_proj.shape[0])
            if pad:
                r2 = torch.nn.functional.pad(r2, (0, 0, 0, pad))
        y = gemm2(hq, hsf, pq, psf, mp, w_proj.shape[0], f, epi=GE_BF16_RES if r2 is not None else GE_BF16, r=r2, bn=bn2)[0]
        ctx.save_for_backward(xq_c, xsf_c, h, hq_c, hsf_c, w_fc, w_proj)
        ctx.has_res, ctx.shp, ctx.ws, ctx.m = residual is not None, shp, (w_fc, w_proj), m
        COUNTS["mlp_mxfp8"] += 1
        return y[:m].view(shp[:-1] + (w_proj.shape[0],))

    @staticmethod
    def backward(ctx, dy):
        xq_c, xsf_c, h, hq_c, hsf_c, w_fc, w_proj = ctx.saved_tensors
        mp, f = h.shape
        c = w_fc.shape[1]
        m = ctx.m
        dy2 = C._c(dy).view(m, -1)
        if mp != m:
            dy2 = torch.nn.functional.pad(dy2, (0, 0, 0, mp - m))
        dyq, dysf, dyq_c, dysf_c = quant2(dy2, col=True, group_c=128)
        bn1, bn2 = bn_for(c, True), bn_for(f)
        ptq, ptsf = weight_q2(w_proj, True, bn1)                    # [f, c]: dh = dy @ w_proj
        _, dpq, dpsf, dpq_c, dpsf_c = gemm2(dyq, dysf, ptq, ptsf, mp, f, c, epi=GE_MUL_2SQRT, r=h, want_d=False, want_q=True,
                                             want_t=True, dt_group=128, bn=bn1)
        g_proj = wgrad2(dyq_c, dysf_c, hq_c, hsf_c, ctx.ws[1])
        ftq, ftsf = weight_q2(w_fc, True, bn2)                      # [c, f]: dx = dpre @ w_fc
        dx = gemm2(dpq, dpsf, ftq, ftsf, mp, c, f, bn=bn2)[0][:m].view(ctx.shp)
        g_fc = wgrad2(dpq_c, dpsf_c, xq_c, xsf_c, ctx.ws[0])
        return dx, g_fc, g_proj, (dy if ctx.has_res else None)


class _MxExpertsFn(torch.autograd.Function):
    """The local experts' ReLU^2 MLPs as batched block-scaled GEMMs over ``[E_local, rows, d]`` (rows grouped by expert):
    the same six GEMMs as the dense MXFP8 MLP with the expert index as the batch axis (reference: ``moe_expert8_mlp``,
    round2/source/train.py:10731, and ``moe8_refresh`` :7309 for the per-step weight pre-cast)."""

    @staticmethod
    def forward(ctx, xs, w_fc, w_proj):
        e, f, d = w_fc.shape
        x3 = C._c(xs).view(e, -1, d)
        rows = x3.shape[1]
        dev = xs.device
        xq, xsf, _, _ = quant2(x3.view(-1, d))                              # rows % 128 == 0: batches are whole chunk runs
        xq_c = torch.empty(e, rows, d, dtype=torch.uint8, device=dev)
        xsf_c = torch.zeros(e, sf2_bytes(d, rows, BN_WGRAD), dtype=torch.uint8, device=dev)
        for j in range(e):
            quant2(x3[j], row=False, col=True, group_c=BN_WGRAD, out=(None, None, xq_c[j], xsf_c[j]))
        bn1, bn2 = bn_for(d, True), bn_for(f)
        wq, wsf = weight_q2_batched(w_fc, False, bn1)
        h, hq, hsf, hq_c, hsf_c = gemm2(xq.view(e, rows, d), xsf, wq, wsf, rows, f, d, epi=GE_RELU2, want_q=True, want_t=True,
                                        dt_group=BN_WGRAD, bn=bn1, batch=e)
        pq, psf = weight_q2_batched(w_proj, False, bn2)
        y = gemm2(hq, hsf, pq, psf, rows, d, f, bn=bn2, batch=e)[0]
        ctx.save_for_backward(xq_c, xsf_c, h, hq_c, hsf_c, w_fc, w_proj)
        ctx.ws = (w_fc, w_proj)
        COUNTS["moe_experts_mxfp8"] += 1
        return y.view(xs.shape)

    @staticmethod
    def backward(ctx, dy):
        xq_c, xsf_c, h, hq_c, hsf_c, w_fc, w_proj = ctx.saved_tensors
        e, f, d = w_fc.shape
        rows = h.shape[1]
        dev = dy.device
        dy3 = C._c(dy).view(e, rows, d)
        dyq, dysf, _, _ = quant2(dy3.view(-1, d))
        dyq_c = torch.empty(e, rows, d, dtype=torch.uint8, device=dev)
        dysf_c = torch.zeros(e, sf2_bytes(d, rows, 128), dtype=torch.uint8, device=dev)
        for j in range(e):
            quant2(dy3[j], row=False, col=True, group_c=128, out=(None, None, dyq_c[j], dysf_c[j]))
        bn1, bn2 = bn_for(d, True), bn_for(f)
        ptq, ptsf = weight_q2_batched(w_proj, True, bn1)                   # [e, f, d]: dh = dy @ w_proj
        _, dpq, dpsf, dpq_c, dpsf_c = gemm2(dyq.view(e, rows, d), dysf, ptq, ptsf, rows, f, d, epi=GE_MUL_2SQRT, r=h, want_d=False,
                                             want_q=True, want_t=True, dt_group=128, bn=bn1, batch=e)
        ftq, ftsf = weight_q2_batched(w_fc, True, bn2)                     # [e, d, f]: dx = dpre @ w_fc
        dx = gemm2(dpq, dpsf, ftq, ftsf, rows, d, f, bn=bn2, batch=e)[0]
        outs = []
        for w, a, asf, b, bsf in ((ctx.ws[0], dpq_c, dpsf_c, xq_c, xsf_c), (ctx.ws[1], dyq_c, dysf_c, hq_c, hsf_c)):
            g = getattr(w, "main_grad", None)
            ret = None
            if g is None:
                g = ret = torch.zeros(w.shape, dtype=torch.float32, device=dev)
            gemm2(a, asf, b, bsf, w.shape[1], w.shape[2], rows, a_major=1, b_major=1, epi=GE_ACC_F32, out=g, bn=BN_WGRAD, batch=e)
            outs.append(ret.to(w.dtype) if ret is not None else None)
        return dx.view(dy.shape), outs[0], outs[1]


def experts_apply(xs, w_fc, w_proj) -> bool:
    e, f, d = w_fc.shape
    rows = xs.numel() // (e * d)
    return xs.dtype == torch.bfloat16 and d % 128 == 0 and f % 128 == 0 and rows % 128 == 0 and rows > 0


def mlp(x, w_fc, w_proj, residual=None):
    if not applies(x, w_fc, w_proj):
        return C._MlpFn.apply(x, w_fc, w_proj, residual)
    return _MxMlpFn.apply(x, w_fc, w_proj, residual)
