"""MXFP8 (OCP microscaling, E4M3 elements, UE8M0 scale per 1 x 32 block) operators on the tcgen05 block-scaled GEMM.

``mlp`` is the fused ReLU^2 MLP: the normalised input is quantised once; the c_fc GEMM's epilogue applies ReLU^2, stores
``h`` in bf16 (kept for the weight gradients) *and* re-quantised along the hidden axis with its block scales, which the
c_proj GEMM consumes directly; the backward's dX GEMMs run in MXFP8 the same way (``dpre = (dy W_proj) * 2 sqrt(h)`` is
re-quantised in the epilogue for the next GEMM); weight gradients stay in bf16 and accumulate into the optimizer slab.

Weights are quantised once per optimizer step, in both orientations (along ``in`` for forward, along ``out`` for dX), and
cached until ``weights_updated()`` is called (reference: the per-step fp8 scale / pre-cast refresh,
``fp8_refresh_weights`` round2/source/train.py:6617-6657, and its per-step quantised-weight caches keyed on an epoch,
round1/source/train.py:2059-2076).
"""
from __future__ import annotations

import ctypes

import torch

from . import COUNTS
from . import _lib as L
from . import cuda as C

_I, _L, _F = ctypes.c_int, ctypes.c_longlong, ctypes.c_float
MX_BF16, MX_BF16_RES, MX_RELU2, MX_MUL_2SQRT = 0, 1, 2, 4
_EPOCH = [0]
_CACHE = {}


def weights_updated():
    """Invalidate every cached quantised weight (call after each optimizer step)."""
    _EPOCH[0] += 1


GROUP_A, GROUP_B = 128, 160       # scale row-group size by operand role (activations / weights)


def sf_bytes(rows: int, k: int, group: int = GROUP_A) -> int:
    return -(-rows // group) * (k // 128) * -(-group // 128) * 512


def quantize(x2: torch.Tensor, group: int = GROUP_A):
    """bf16 ``[R, K]`` (K a multiple of 128) -> ``(q uint8 [R, K], scales uint8 [sf_bytes])`` quantised along K.
    ``group`` selects the scale layout: ``GROUP_A`` for the GEMM's A operand, ``GROUP_B`` for its B operand."""
    r, k = x2.shape
    q = torch.empty(r, k, dtype=torch.uint8, device=x2.device)
    sf = torch.zeros(sf_bytes(r, k, group), dtype=torch.uint8, device=x2.device)
    L.call("bones_mx_quant_rows", L.ptr(x2), _L(x2.stride(0)), L.ptr(q), _L(k), L.ptr(sf), _L(r), _L(k), _I(group),
           L.stream())
    COUNTS["mx_quant"] += 1
    return q, sf


def weight_q(w: torch.Tensor, transposed: bool):
    """Quantised weight for ``x @ w.T`` (``transposed=False``: along ``in``) or ``dy @ w`` (``True``: ``w.T`` along ``out``)."""
    key = (w.data_ptr(), tuple(w.shape), transposed)
    ent = _CACHE.get(key)
    if ent is None or ent[0] != _EPOCH[0] or ent[1] != w._version:
        src = w.detach().t().contiguous() if transposed else w.detach()
        ent = (_EPOCH[0], w._version) + quantize(src, GROUP_B)
        _CACHE[key] = ent
    return ent[2], ent[3]


def gemm(aq, sfa, bq, sfb, m, n, k, *, epi=MX_BF16, r=None, beta=1.0, want_q=False):
    d = torch.empty(m, n, dtype=torch.bfloat16, device=aq.device)
    dq = dsf = None
    if want_q:
        dq = torch.empty(m, n, dtype=torch.uint8, device=aq.device)
        dsf = torch.zeros(sf_bytes(m, n), dtype=torch.uint8, device=aq.device)
    L.call("bones_gemm_mxfp8", L.ptr(aq), L.ptr(sfa), L.ptr(bq), L.ptr(sfb), L.ptr(d), L.ptr(r), L.ptr(dq), L.ptr(dsf), _I(m),
           _I(n), _I(k), _L(n), _L(r.stride(0) if r is not None else 0), _I(epi), _F(beta), L.stream())
    COUNTS["mx_gemm"] += 1
    return (d, dq, dsf) if want_q else d


def linear(x2: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """``x2 @ w.T`` with both operands block-quantised along K."""
    xq, xsf = quantize(x2)
    wq, wsf = weight_q(w, False)
    return gemm(xq, xsf, wq, wsf, x2.shape[0], w.shape[0], x2.shape[1])


def applies(x, w_fc, w_proj) -> bool:
    c, f = w_fc.shape[1], w_fc.shape[0]
    return x.dtype == torch.bfloat16 and c % 128 == 0 and f % 128 == 0


class _MxMlpFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w_fc, w_proj, residual):
        shp = x.shape
        x2 = C._c(x).view(-1, shp[-1])
        m, c = x2.shape
        f = w_fc.shape[0]
        xq, xsf = quantize(x2)
        wq, wsf = weight_q(w_fc, False)
        h, hq, hsf = gemm(xq, xsf, wq, wsf, m, f, c, epi=MX_RELU2, want_q=True)
        pq, psf = weight_q(w_proj, False)
        r2 = C._c(residual).view(-1, w_proj.shape[0]) if residual is not None else None
        y = gemm(hq, hsf, pq, psf, m, w_proj.shape[0], f, epi=MX_BF16_RES if r2 is not None else MX_BF16, r=r2)
        ctx.save_for_backward(x2, h, w_fc, w_proj)
        ctx.has_res, ctx.shp, ctx.ws = residual is not None, shp, (w_fc, w_proj)
        COUNTS["mlp_mxfp8"] += 1
        return y.view(shp[:-1] + (w_proj.shape[0],))

    @staticmethod
    def backward(ctx, dy):
        x2, h, w_fc, w_proj = ctx.saved_tensors
        m, c = x2.shape
        f = w_fc.shape[0]
        dy2 = C._c(dy).view(m, -1)
        dyq, dysf = quantize(dy2)
        ptq, ptsf = weight_q(w_proj, True)                   # [f, c]: dh = dy @ w_proj
        dpre, dpq, dpsf = gemm(dyq, dysf, ptq, ptsf, m, f, c, epi=MX_MUL_2SQRT, r=h, want_q=True)
        (g_proj,) = C._wgrad(dy2, h, (ctx.ws[1],))
        ftq, ftsf = weight_q(w_fc, True)                     # [c, f]: dx = dpre @ w_fc
        dx = gemm(dpq, dpsf, ftq, ftsf, m, c, f).view(ctx.shp)
        (g_fc,) = C._wgrad(dpre, x2, (ctx.ws[0],))
        return dx, g_fc, g_proj, (dy if ctx.has_res else None)


def mlp(x, w_fc, w_proj, residual=None):
    if not applies(x, w_fc, w_proj):
        return C._MlpFn.apply(x, w_fc, w_proj, residual)
    return _MxMlpFn.apply(x, w_fc, w_proj, residual)
