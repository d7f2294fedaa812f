"""Native (sm_100a) operator bodies: autograd ``Function``s around the C entry points of ``libbones_b200.so``.

Conventions: activations are bf16, contiguous, flattened to ``[M, C]``; weights are bf16 replicas ``[out, in]``.  A weight
that carries ``main_grad`` (the optimizer's fp32 reduce-scatter slab view) receives its gradient by accumulation inside
the weight-gradient GEMM's epilogue and autograd sees ``None`` for it (reference: dW written straight into the
optimizer's buffer, ``GradFoldIn`` round2/source/train.py:4677-4723 and ``_LinearAccum`` round1/source/train.py:8484).
"""
from __future__ import annotations

import ctypes
import os

import torch
import torch.nn.functional as F

from . import _lib as L
from . import COUNTS

_I, _L, _F = ctypes.c_int, ctypes.c_longlong, ctypes.c_float
BF16 = torch.bfloat16
_LIBRARY_OPS = os.environ.get("BONES_LIBRARY_OPS", "0") not in ("0", "", "false")


def _c(t):
    return t if t.is_contiguous() else t.contiguous()


def _fused_rows(ws):
    """If the tensors are adjacent row blocks of one storage return a single ``[sum rows, cols]`` view, else None."""
    w0 = ws[0]
    cols = w0.shape[1]
    off = w0.storage_offset()
    for w in ws:
        if (w.dtype != w0.dtype or w.shape[1] != cols or not w.is_contiguous() or w.storage_offset() != off
                or w.untyped_storage().data_ptr() != w0.untyped_storage().data_ptr()):
            return None
        off += w.numel()
    rows = sum(w.shape[0] for w in ws)
    return torch.empty(0, dtype=w0.dtype, device=w0.device).set_(w0.untyped_storage(), w0.storage_offset(), (rows, cols),
                                                                 (cols, 1))


# -- GEMM helpers (2-D, row-major tensors) -----------------------------------------------------------------------
def mm_nt(x, w, out=None, epi=L.EPI_BF16, r=None, alpha=1.0, beta=1.0, out_dtype=BF16):
    """``x [M,K] @ w[N,K]^T``"""
    m, k = x.shape
    n = w.shape[0]
    out = out if out is not None else torch.empty(m, n, dtype=out_dtype, device=x.device)
    L.gemm(x, w, out, m=m, n=n, k=k, lda=x.stride(0), ldb=w.stride(0), ldd=out.stride(0), epi=epi, r=r,
           ldr=r.stride(0) if r is not None else 0, alpha=alpha, beta=beta)
    COUNTS["gemm"] += 1
    return out


def mm_nn(x, w, out=None, epi=L.EPI_BF16, r=None, alpha=1.0, beta=1.0):
    """``x [M,N] @ w[N,K]`` (w row-major: the contraction index is w's row -> MN-major B operand)"""
    m, n = x.shape
    k = w.shape[1]
    out = out if out is not None else torch.empty(m, k, dtype=BF16, device=x.device)
    L.gemm(x, w, out, m=m, n=k, k=n, lda=x.stride(0), ldb=w.stride(0), ldd=out.stride(0), b_major=1, epi=epi, r=r,
           ldr=r.stride(0) if r is not None else 0, alpha=alpha, beta=beta)
    COUNTS["gemm"] += 1
    return out


def mm_nn_acc(x, w, out32):
    """``out32 [M,K] (fp32) += x[M,N] @ w[N,K]``: the fp32 accumulate form lets a long contraction over few output tiles be
    split across the SMs (split-K with vector atomics)"""
    m, n = x.shape
    k = w.shape[1]
    L.gemm(x, w, out32, m=m, n=k, k=n, lda=x.stride(0), ldb=w.stride(0), ldd=out32.stride(0), b_major=1, epi=L.EPI_ACC_F32)
    COUNTS["gemm"] += 1
    return out32


def mm_tn_acc(dy, x, grad, alpha=1.0, push_ptr=None):
    """``grad [N,K] (fp32) += alpha * dy[M,N]^T @ x[M,K]`` (both operands MN-major: contraction over rows).
    ``push_ptr``: device address of the same gradient buffer on the GPU that owns this matrix; the GEMM epilogue then
    adds its tiles there with vector atomics over NVLink, which is the reduce-scatter of the data-parallel gradient done
    tile by tile inside the weight-gradient GEMM."""
    m, n = dy.shape
    k = x.shape[1]
    L.gemm(dy, x, grad, m=n, n=k, k=m, lda=dy.stride(0), ldb=x.stride(0), ldd=grad.stride(0), a_major=1, b_major=1,
           epi=L.EPI_ACC_F32, alpha=alpha, d_ptr=push_ptr, atomic=push_ptr is not None)
    COUNTS["gemm"] += 1
    return grad


def _wgrad(dy2, x2, ws):
    """Weight gradient for one or several row-adjacent weights.  Returns the tuple autograd expects."""
    grads = [getattr(w, "main_grad", None) for w in ws]
    if all(g is not None for g in grads):
        push = [getattr(w, "main_grad_push", None) for w in ws]       # owner-side addresses (fused reduce-scatter)
        fused = _fused_rows(grads) if len(grads) > 1 else grads[0]
        if all(p is not None for p in push):
            # one GEMM when the weights are adjacent in the owner's buffer too (same owner), else one per weight
            adjacent = all(push[j + 1] == push[j] + grads[j].numel() * 4 for j in range(len(ws) - 1))
            if fused is not None and adjacent:
                mm_tn_acc(dy2, x2, fused, push_ptr=push[0])
            else:
                o = 0
                for w, g, pp in zip(ws, grads, push):
                    mm_tn_acc(dy2[:, o:o + w.shape[0]], x2, g, push_ptr=pp)
                    o += w.shape[0]
        elif fused is not None:
            mm_tn_acc(dy2, x2, fused)
        else:
            o = 0
            for w, g in zip(ws, grads):
                mm_tn_acc(dy2[:, o:o + w.shape[0]], x2, g)
                o += w.shape[0]
        return tuple(None for _ in ws)
    full = torch.zeros(dy2.shape[1], x2.shape[1], dtype=torch.float32, device=x2.device)
    mm_tn_acc(dy2, x2, full)
    outs, o = [], 0
    for w in ws:
        outs.append(full[o:o + w.shape[0]].to(w.dtype))
        o += w.shape[0]
    return tuple(outs)


class _LinearFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, residual, *ws):
        shp = x.shape
        x2 = _c(x).view(-1, shp[-1])
        w = _fused_rows(ws) if len(ws) > 1 else ws[0]
        if w is None:
            w = torch.cat(ws, 0)
        r2 = _c(residual).view(-1, w.shape[0]) if residual is not None else None
        y = mm_nt(x2, w, epi=L.EPI_BF16_RES if r2 is not None else L.EPI_BF16, r=r2)
        ctx.save_for_backward(x2, w)
        ctx.ws, ctx.has_res, ctx.shp = ws, residual is not None, shp
        return y.view(*shp[:-1], w.shape[0])

    @staticmethod
    def backward(ctx, dy):
        x2, w = ctx.saved_tensors
        dy2 = _c(dy).view(-1, w.shape[0])
        dx = mm_nn(dy2, w).view(ctx.shp) if ctx.needs_input_grad[0] else None
        gws = _wgrad(dy2, x2, ctx.ws)
        return (dx, dy if ctx.has_res else None) + gws


def _mx_linear_ok(x, ws):
    return (x.dtype == BF16 and x.shape[-1] % 128 == 0 and all(w.shape[0] % 128 == 0 for w in ws)
            and not any(getattr(w, "main_grad_push", None) is not None for w in ws))


def linear(x, w, residual=None, precision="bf16"):
    if precision == "mxfp8" and _mx_linear_ok(x, (w,)):
        from . import mxfp8
        return mxfp8._MxLinearFn.apply(x, residual, w)
    return _LinearFn.apply(x, residual, w)


def linear_qkv(x, wq, wk, wv, precision="bf16"):
    if precision == "mxfp8" and _mx_linear_ok(x, (wq, wk, wv)):
        from . import mxfp8
        return mxfp8._MxLinearFn.apply(x, None, wq, wk, wv)
    return _LinearFn.apply(x, None, wq, wk, wv)


class _MlpFn(torch.autograd.Function):
    """c_fc GEMM with ReLU^2 epilogue, c_proj GEMM with residual epilogue.  Only ``h = relu(pre)^2`` is kept; the
    backward recovers ``relu(pre) = sqrt(h)`` inside the dX GEMM's epilogue (reference: ``relu2 bwd_from_h``,
    round1/source/train.py:537)."""

    @staticmethod
    def forward(ctx, x, w_fc, w_proj, residual):
        shp = x.shape
        x2 = _c(x).view(-1, shp[-1])
        h = mm_nt(x2, w_fc, epi=L.EPI_RELU2)
        r2 = _c(residual).view(-1, w_proj.shape[0]) if residual is not None else None
        y = mm_nt(h, w_proj, epi=L.EPI_BF16_RES if r2 is not None else L.EPI_BF16, r=r2)
        ctx.save_for_backward(x2, h, w_fc, w_proj)
        ctx.has_res, ctx.shp = residual is not None, shp
        ctx.ws = (w_fc, w_proj)
        COUNTS["mlp"] += 1
        return y.view(shp[:-1] + (w_proj.shape[0],))

    @staticmethod
    def backward(ctx, dy):
        x2, h, w_fc, w_proj = ctx.saved_tensors
        dy2 = _c(dy).view(-1, w_proj.shape[0])
        dpre = mm_nn(dy2, w_proj, epi=L.EPI_MUL_2SQRT, r=h)
        (g_proj,) = _wgrad(dy2, h, (ctx.ws[1],))
        dx = mm_nn(dpre, w_fc).view(ctx.shp)
        (g_fc,) = _wgrad(dpre, x2, (ctx.ws[0],))
        return dx, g_fc, g_proj, (dy if ctx.has_res else None)


def mlp(x, w_fc, w_proj, residual=None, precision="bf16"):
    if precision == "mxfp8":
        from . import mxfp8
        return mxfp8.mlp(x, w_fc, w_proj, residual)
    return _MlpFn.apply(x, w_fc, w_proj, residual)


# -- norms ---------------------------------------------------------------------------------------------------------
class _RmsNormFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x):
        x2 = _c(x).view(-1, x.shape[-1])
        y = torch.empty_like(x2)
        L.call("bones_rmsnorm_fwd", L.ptr(x2), L.ptr(y), _I(x2.shape[0]), _I(x2.shape[1]), L.stream())
        ctx.save_for_backward(x2)
        COUNTS["rmsnorm"] += 1
        return y.view(x.shape)

    @staticmethod
    def backward(ctx, dy):
        (x2,) = ctx.saved_tensors
        dy2 = _c(dy).view(x2.shape)
        dx = torch.empty_like(x2)
        L.call("bones_rmsnorm_bwd", L.ptr(x2), L.ptr(dy2), L.ptr(None), L.ptr(dx), _I(x2.shape[0]), _I(x2.shape[1]),
               L.stream())
        return dx.view(dy.shape)


def rms_norm(x):
    if x.dtype != BF16:
        from ..ref import functional as RF
        return RF.rms_norm(x)
    if _LIBRARY_OPS:
        from . import registry
        COUNTS["rmsnorm"] += 1
        return registry.rms_norm(x)
    return _RmsNormFn.apply(x)


class _NormSplitFn(torch.autograd.Function):
    """``x -> (x, rms_norm(x))`` for the ``x + f(norm(x))`` pattern: the backward adds the gradient of the pass-through
    copy inside the norm-backward kernel instead of leaving a separate accumulation to autograd."""

    @staticmethod
    def forward(ctx, x):
        x2 = _c(x).view(-1, x.shape[-1])
        y = torch.empty_like(x2)
        L.call("bones_rmsnorm_fwd", L.ptr(x2), L.ptr(y), _I(x2.shape[0]), _I(x2.shape[1]), L.stream())
        ctx.save_for_backward(x2)
        COUNTS["rmsnorm"] += 1
        return x.view(x.shape), y.view(x.shape)

    @staticmethod
    def backward(ctx, dx_pass, dy):
        (x2,) = ctx.saved_tensors
        if dy is None:
            return dx_pass
        dy2 = _c(dy).view(x2.shape)
        add = _c(dx_pass).view(x2.shape) if dx_pass is not None else None
        dx = torch.empty_like(x2)
        L.call("bones_rmsnorm_bwd", L.ptr(x2), L.ptr(dy2), L.ptr(add), L.ptr(dx), _I(x2.shape[0]), _I(x2.shape[1]), L.stream())
        return dx.view(dy.shape)


def norm_split(x):
    if x.dtype != BF16:
        from ..ref import functional as RF
        return x, RF.rms_norm(x)
    return _NormSplitFn.apply(x)


class X0Accum:
    """Shared by the blocks of one forward pass: their backward passes add the gradient of the common ``x0`` operand into
    one buffer inside the kernel, and the first block (the last to run backward) hands the sum to autograd."""

    def __init__(self):
        self.pending = 0
        self.buf = None


class _ResidMixNormFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, x0, a, b, acc=None):
        ctx.acc = acc
        if acc is not None:
            acc.pending += 1
        x2, x02 = _c(x).view(-1, x.shape[-1]), _c(x0).view(-1, x.shape[-1])
        xm, xn = torch.empty_like(x2), torch.empty_like(x2)
        af, bf = a.detach().float().reshape(1), b.detach().float().reshape(1)
        L.call("bones_resid_mix_norm_fwd", L.ptr(x2), L.ptr(x02), L.ptr(af), L.ptr(bf), L.ptr(xm), L.ptr(xn),
               _I(x2.shape[0]), _I(x2.shape[1]), L.stream())
        ctx.save_for_backward(x2, x02, xm, af, bf)
        ctx.shape = x.shape
        COUNTS["resid_mix_norm"] += 1
        return xm.view(x.shape), xn.view(x.shape)

    @staticmethod
    def backward(ctx, dxm, dxn):
        x2, x02, xm, af, bf = ctx.saved_tensors
        if dxm is None:
            dxm = torch.zeros_like(xm)
        if dxn is None:
            dxn = torch.zeros_like(xm)
        dxm2, dxn2 = _c(dxm).view(x2.shape), _c(dxn).view(x2.shape)
        acc = ctx.acc
        dx = torch.empty_like(x2)
        accumulate = acc is not None and acc.buf is not None
        dx0 = acc.buf if accumulate else torch.empty_like(x2)
        dab = torch.zeros(2, dtype=torch.float32, device=x2.device)
        L.call("bones_resid_mix_norm_bwd", L.ptr(x2), L.ptr(x02), L.ptr(xm), L.ptr(af), L.ptr(bf), L.ptr(dxm2),
               L.ptr(dxn2), L.ptr(dx), L.ptr(dx0), L.ptr(dab[0:1]), L.ptr(dab[1:2]), _I(x2.shape[0]), _I(x2.shape[1]),
               _I(int(accumulate)), L.stream())
        if acc is not None:
            acc.buf = dx0
            acc.pending -= 1
            if acc.pending > 0:
                return dx.view(ctx.shape), None, dab[0:1], dab[1:2], None
            acc.buf = None
        return dx.view(ctx.shape), dx0.view(ctx.shape), dab[0:1], dab[1:2], None


def resid_mix_norm(x, x0, a, b, acc=None):
    return _ResidMixNormFn.apply(x, x0, a, b, acc)


# -- embedding -------------------------------------------------------------------------------------------------------
class _EmbeddingFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, idx, weight):
        flat = _c(idx).view(-1)
        out = torch.empty(flat.numel(), weight.shape[1], dtype=weight.dtype, device=weight.device)
        L.call("bones_gather_rows", L.ptr(weight), L.ptr(flat), _I(int(flat.dtype == torch.int64)), L.ptr(out),
               _I(flat.numel()), _I(weight.shape[1]), _L(weight.shape[0]), L.stream())
        ctx.save_for_backward(flat)
        ctx.weight = weight
        COUNTS["embedding"] += 1
        return out.view(*idx.shape, weight.shape[1])

    @staticmethod
    def backward(ctx, dy):
        (flat,) = ctx.saved_tensors
        w = ctx.weight
        grad = getattr(w, "main_grad", None)
        ret = None
        if grad is None:
            grad = torch.zeros(w.shape, dtype=torch.float32, device=w.device)
            ret = grad
        dy2 = _c(dy).view(-1, w.shape[1])
        L.call("bones_scatter_add_rows", L.ptr(dy2), L.ptr(flat), _I(int(flat.dtype == torch.int64)), L.ptr(grad),
               _I(flat.numel()), _I(w.shape[1]), _L(w.shape[0]), L.stream())
        return None, (ret.to(w.dtype) if ret is not None else None)


def embedding(idx, weight, dtype):
    if weight.dtype != BF16:
        return F.embedding(idx, weight).to(dtype)
    return _EmbeddingFn.apply(idx, weight)


# -- attention -------------------------------------------------------------------------------------------------------
def attention(qkv, cos, sin, n_head, head_dim, scale, doc_start, window):
    """RoPE + QK-norm + causal (document-reset, optionally banded) attention on the tcgen05 flash-attention kernels
    (``csrc/attention.cu``, ``csrc/attention_bwd_split.cu``).  A shape the kernels do not cover raises: the SDPA route
    exists only as the explicit baseline (``BONES_KERNELS=ref``), never as a silent fallback (reference: a kernel
    route that does not apply on the device raises, round2/source/train.py:4882-4887)."""
    from . import attention_native as AN
    t = qkv.shape[1]
    pad = -t % 128
    if pad:
        # the kernels work on 128-token tiles: a ragged length (scoring, cache-free decoding) is zero-padded at the end,
        # which causal masking keeps away from the real positions, and the padding rows are dropped again
        qkv = F.pad(qkv, (0, 0, 0, pad))
        cos, sin = F.pad(cos, (0, 0, 0, pad)), F.pad(sin, (0, 0, 0, pad))
        if doc_start is not None:
            doc_start = F.pad(doc_start, (0, pad), value=t)
    why = AN.why_not(qkv, n_head, head_dim, window)
    if why:
        raise ValueError(f"native attention does not cover this call: {why}")
    COUNTS["attention"] += 1
    if _LIBRARY_OPS and head_dim == 128:             # the same kernels behind torch.library custom ops (ops/registry.py)
        from . import registry
        y = registry.attention(qkv, cos, sin, n_head, head_dim, scale, doc_start, window)
    else:
        y = AN.attention(qkv, cos, sin, n_head, head_dim, scale, doc_start, window)
    return y[:, :t] if pad else y


# -- loss head -------------------------------------------------------------------------------------------------------
LOSS_ROWS = max(128, int(os.environ.get("BONES_LOSS_ROWS", 4096)))       # rows per logits block


class _LmHeadLossFn(torch.autograd.Function):
    """Chunked head: for each block of rows the logits GEMM, the softcap cross-entropy (which overwrites the logits
    with their gradient), the dX GEMM and the dW GEMM (accumulating into the head's gradient slab) run back to back, so
    only one ``[rows, V]`` block of logits ever exists and no logits are recomputed in backward.  The loss is the mean
    over valid targets divided by ``loss_div`` (reference: ``chunked_loss_mean`` round2/source/train.py:6364-6391 and
    ``loss_scaled`` :11712)."""

    @staticmethod
    def forward(ctx, x, w, targets, vocab, cap, loss_div, row_weights, want_grad, aux=None, label_smoothing=0.0):
        # aux: up to two (targets, absolute row weights) pairs that share the row's soft-max (multi-token prediction)
        shp = x.shape
        x2 = _c(x).view(-1, shp[-1])
        m = x2.shape[0]
        tg = _c(targets).view(-1).to(torch.int64)
        nll = torch.empty(m, dtype=torch.float32, device=x.device)
        n_valid = (tg >= 0).sum().float().reshape(1)
        # dX contracts over the whole vocabulary into few output tiles: accumulated in fp32 so the contraction can be split
        dx32 = torch.zeros(x2.shape, dtype=torch.float32, device=x.device) if want_grad else None
        rw = _c(row_weights).view(-1).float() if row_weights is not None else None
        vp = w.shape[0]
        grad_w = getattr(w, "main_grad", None)
        own_gw = None
        if want_grad and grad_w is None:
            own_gw = grad_w = torch.zeros(w.shape, dtype=torch.float32, device=w.device)
        buf = torch.empty(min(LOSS_ROWS, m), vp, dtype=BF16, device=x.device)
        aux = [(_c(t).view(-1).to(torch.int64), _c(wk).view(-1).float()) for t, wk in (aux or [])][:2]
        nll_aux = torch.zeros(m, dtype=torch.float32, device=x.device) if aux else None

        def aux_ptrs(r0, r1):
            out = []
            for k in range(2):
                out += [L.ptr(aux[k][0][r0:r1]), L.ptr(aux[k][1][r0:r1])] if k < len(aux) else [L.ptr(None), L.ptr(None)]
            return out + [L.ptr(nll_aux[r0:r1] if aux else None)]

        for r0 in range(0, m, LOSS_ROWS):
            r1 = min(m, r0 + LOSS_ROWS)
            lg = buf[:r1 - r0]
            # the logits GEMM soft-caps in its epilogue (cap * tanh(. / cap)); the loss kernel then only exponentiates
            mm_nt(x2[r0:r1], w, out=lg, epi=L.EPI_SOFTCAP, alpha=1.0 / cap, beta=cap)
            L.call("bones_softcap_ce", L.ptr(lg), _L(vp), L.ptr(tg[r0:r1]), _I(vocab), _F(cap), L.ptr(nll[r0:r1]),
                   L.ptr(lg if want_grad else None), L.ptr(rw[r0:r1] if rw is not None else None), L.ptr(n_valid),
                   _F(1.0 / loss_div), _I(r1 - r0), _I(1), *aux_ptrs(r0, r1), _F(label_smoothing), L.stream())
            if want_grad:
                mm_nn_acc(lg, w, dx32[r0:r1])
                mm_tn_acc(lg, x2[r0:r1], grad_w)
        COUNTS["lmhead_loss"] += 1
        dx = dx32.to(x2.dtype) if want_grad else None
        ctx.dx, ctx.shp, ctx.own_gw, ctx.wdtype = dx, shp, own_gw, w.dtype
        if rw is not None:
            loss = (nll * rw).sum()
        else:
            loss = nll.sum() / n_valid.clamp_min(1.0)[0] / loss_div
        if aux:
            loss = loss + nll_aux.sum()
        ctx.mark_non_differentiable(nll)
        return loss, nll

    @staticmethod
    def backward(ctx, dloss, _dnll):
        dx = ctx.dx.view(ctx.shp) * dloss.to(ctx.dx.dtype)
        gw = ctx.own_gw.to(ctx.wdtype) * dloss.to(ctx.wdtype) if ctx.own_gw is not None else None
        return dx, gw, None, None, None, None, None, None, None, None


def lmhead_loss(x, w, targets, vocab, cap, reduction="mean", row_weights=None, loss_div=1.0, aux=None, label_smoothing=0.0):
    want_grad = torch.is_grad_enabled() and (x.requires_grad or w.requires_grad) and reduction == "mean"
    loss, nll = _LmHeadLossFn.apply(x, w, targets, vocab, cap, float(loss_div), row_weights, want_grad, aux,
                                    float(label_smoothing))
    if reduction == "mean":
        return loss
    if reduction == "sum":
        return nll.sum()
    return nll.view(targets.shape)


def lmhead_logits(x, w, vocab, cap):
    shp = x.shape
    x2 = _c(x).view(-1, shp[-1])
    lg = mm_nt(x2, w)
    out = torch.empty(x2.shape[0], vocab, dtype=torch.float32, device=x.device)
    L.call("bones_softcap_logits", L.ptr(lg), _L(w.shape[0]), L.ptr(out), _I(vocab), _F(cap), _L(x2.shape[0]), L.stream())
    return out.view(*shp[:-1], vocab)


# -- output-side hashed table ----------------------------------------------------------------------------------------
def os1_apply_signs(x, hsign, out_dtype=None):
    """``signs(hsign) * x`` for rows ``x [n, dim]`` (bf16 or fp32) and sign hashes ``hsign [n]`` int64."""
    x = _c(x)
    out_dtype = out_dtype or x.dtype
    kind = {(BF16, BF16): 0, (torch.float32, torch.float32): 1, (torch.float32, BF16): 2}[(x.dtype, out_dtype)]
    out = torch.empty(x.shape, dtype=out_dtype, device=x.device)
    L.call("bones_os1_signs", L.ptr(x), L.ptr(_c(hsign)), L.ptr(out), _L(x.shape[0]), _I(x.shape[1]), _I(kind), L.stream())
    return out


def os1_gate_dot(u, code, nxt, a0):
    """``sd[i] = u[i] . code[nxt[i]] / a0`` (0 where ``nxt[i] < 0``), fp32."""
    sd = torch.empty(u.shape[0], dtype=torch.float32, device=u.device)
    L.call("bones_os1_gate_dot", L.ptr(_c(u)), L.ptr(code), L.ptr(_c(nxt)), L.ptr(sd), _L(u.shape[0]), _I(u.shape[1]),
           _F(1.0 / a0), L.stream())
    return sd


def os1_row_step(table, rows, g, lr, eps, cap):
    """In place on ``table[rows]``: the normalised step and the row budget.  Returns the count of rows the budget scaled
    (a device int32 scalar)."""
    capped = torch.zeros(1, dtype=torch.int32, device=table.device)
    L.call("bones_os1_row_step", L.ptr(table), L.ptr(_c(rows)), L.ptr(_c(g)), _I(rows.numel()), _I(table.shape[1]), _F(lr),
           _F(eps), _F(cap * lr), L.ptr(capped), _I(int(table.dtype == torch.float32)), L.stream())
    return capped


class _LmHeadLossOs1Fn(torch.autograd.Function):
    """The chunked loss head with the output table's read-out: per block of rows the logits GEMM, the scores GEMM
    ``S = U C^T / a0``, one element-wise kernel that adds ``glin S + G k relu(S - thr)`` and soft-caps, the
    cross-entropy kernel (logits overwritten by their gradient), then dX, dW and ``dU = (glin / a0) dLogits C``
    (reference: the OS1-fused loss-head pair, round2/source/train.py:5881-5957 and :6461-6501)."""

    @staticmethod
    def forward(ctx, x, w, u, code, gate, targets, vocab, cap, loss_div, row_weights, want_grad, a0, glin, kthr, thr):
        shp = x.shape
        x2 = _c(x).view(-1, shp[-1])
        u2 = _c(u).view(-1, u.shape[-1])
        m = x2.shape[0]
        tg = _c(targets).view(-1).to(torch.int64)
        gt = _c(gate).view(-1).float()
        nll = torch.empty(m, dtype=torch.float32, device=x.device)
        n_valid = (tg >= 0).sum().float().reshape(1)
        dx32 = torch.zeros(x2.shape, dtype=torch.float32, device=x.device) if want_grad else None
        du32 = torch.zeros(u2.shape, dtype=torch.float32, device=x.device) if want_grad else None
        rw = _c(row_weights).view(-1).float() if row_weights is not None else None
        vp = w.shape[0]
        grad_w = getattr(w, "main_grad", None)
        own_gw = None
        if want_grad and grad_w is None:
            own_gw = grad_w = torch.zeros(w.shape, dtype=torch.float32, device=w.device)
        rows = min(LOSS_ROWS, m)
        buf = torch.empty(rows, vp, dtype=BF16, device=x.device)
        sbuf = torch.empty(rows, vp, dtype=BF16, device=x.device)
        null = L.ptr(None)
        for r0 in range(0, m, LOSS_ROWS):
            r1 = min(m, r0 + LOSS_ROWS)
            lg, sc = buf[:r1 - r0], sbuf[:r1 - r0]
            mm_nt(x2[r0:r1], w, out=lg)
            mm_nt(u2[r0:r1], code, out=sc, alpha=1.0 / a0)
            L.call("bones_os1_combine", L.ptr(lg), L.ptr(sc), L.ptr(gt[r0:r1]), _L(r1 - r0), _I(vp), _L(vp), _F(cap), _F(glin),
                   _F(kthr), _F(thr), _I(1), L.stream())
            L.call("bones_softcap_ce", L.ptr(lg), _L(vp), L.ptr(tg[r0:r1]), _I(vocab), _F(cap), L.ptr(nll[r0:r1]),
                   L.ptr(lg if want_grad else None), L.ptr(rw[r0:r1] if rw is not None else None), L.ptr(n_valid),
                   _F(1.0 / loss_div), _I(r1 - r0), _I(1), null, null, null, null, null, _F(0.0), L.stream())
            if want_grad:
                mm_nn_acc(lg, w, dx32[r0:r1])
                mm_tn_acc(lg, x2[r0:r1], grad_w)
                mm_nn_acc(lg, code, du32[r0:r1])
        COUNTS["lmhead_loss_os1"] += 1
        ctx.dx = dx32.to(x2.dtype) if want_grad else None
        ctx.du = (du32 * (glin / a0)) if want_grad else None
        ctx.shp, ctx.ushp, ctx.own_gw, ctx.wdtype, ctx.udtype = shp, u.shape, own_gw, w.dtype, u.dtype
        if rw is not None:
            loss = (nll * rw).sum()
        else:
            loss = nll.sum() / n_valid.clamp_min(1.0)[0] / loss_div
        ctx.mark_non_differentiable(nll)
        return loss, nll

    @staticmethod
    def backward(ctx, dloss, _dnll):
        dx = ctx.dx.view(ctx.shp) * dloss.to(ctx.dx.dtype)
        du = (ctx.du.view(ctx.ushp) * dloss.float()).to(ctx.udtype)
        gw = ctx.own_gw.to(ctx.wdtype) * dloss.to(ctx.wdtype) if ctx.own_gw is not None else None
        return (dx, gw, du) + (None,) * 12


def lmhead_loss_os1(x, w, targets, vocab, cap, u, code, gate, a0, glin, beta, thr, reduction="mean", row_weights=None,
                    loss_div=1.0):
    want_grad = torch.is_grad_enabled() and (x.requires_grad or w.requires_grad or u.requires_grad) and reduction == "mean"
    loss, nll = _LmHeadLossOs1Fn.apply(x, w, u, code, gate, targets, vocab, cap, float(loss_div), row_weights, want_grad,
                                       float(a0), float(glin), float(beta / (1.0 - thr)), float(thr))
    if reduction == "mean":
        return loss
    if reduction == "sum":
        return nll.sum()
    return nll.view(targets.shape)


def lmhead_logits_os1(x, w, vocab, cap, u, code, gate, a0, glin, beta, thr):
    shp = x.shape
    x2 = _c(x).view(-1, shp[-1])
    u2 = _c(u).view(-1, u.shape[-1])
    vp = w.shape[0]
    lg = mm_nt(x2, w)
    sc = mm_nt(u2, code, alpha=1.0 / a0)
    L.call("bones_os1_combine", L.ptr(lg), L.ptr(sc), L.ptr(_c(gate).view(-1).float()), _L(x2.shape[0]), _I(vp), _L(vp),
           _F(cap), _F(glin), _F(beta / (1.0 - thr)), _F(thr), _I(0), L.stream())
    out = torch.empty(x2.shape[0], vocab, dtype=torch.float32, device=x.device)
    L.call("bones_softcap_logits", L.ptr(lg), _L(vp), L.ptr(out), _I(vocab), _F(cap), _L(x2.shape[0]), L.stream())
    return out.view(*shp[:-1], vocab)


# -- MoE -------------------------------------------------------------------------------------------------------------
class _RouterFn(torch.autograd.Function):
    """Router logits ``h [T, C] @ R[E, C]^T`` in fp32 on the tcgen05 GEMM.  ``E`` (16) is far below a tensor-core tile, so
    the router is padded to 128 rows: the padding costs a few GFLOP, while the library route this replaces converted the
    whole activation to fp32 and ran SIMT fp32 GEMMs (a fifth of an MoE layer's non-GEMM time).  Inputs are the exact
    bf16 values and the accumulation is fp32, which is what ``F.linear(h.float(), R.float())`` computes (reference: the
    fp32 router, round2/source/train.py:11023)."""

    @staticmethod
    def forward(ctx, h, router):
        e, c = router.shape
        rp = torch.zeros(128, c, dtype=BF16, device=h.device)
        rp[:e].copy_(router.detach())
        out = mm_nt(h, rp, epi=L.EPI_F32, out_dtype=torch.float32)
        ctx.save_for_backward(h, rp)
        ctx.e, ctx.rdtype = e, router.dtype
        COUNTS["moe_router"] += 1
        return out[:, :e].contiguous()

    @staticmethod
    def backward(ctx, dl):
        h, rp = ctx.saved_tensors
        t, c = h.shape
        dlp = torch.zeros(t, 128, dtype=BF16, device=h.device)
        dlp[:, :ctx.e].copy_(dl)
        dh = mm_nn(dlp, rp)
        dr32 = torch.zeros(128, c, dtype=torch.float32, device=h.device)
        mm_tn_acc(dlp, h, dr32)
        return dh, dr32[:ctx.e].to(ctx.rdtype)


def router_logits(h, router):
    if h.dtype != BF16 or router.shape[0] > 128 or h.shape[1] % 8:
        return F.linear(h.float(), router.float())
    return _RouterFn.apply(_c(h), router)


def moe_slots(idx, b, t, n_exp, cap):
    """Native capacity slotting: ``idx [b*t, k]`` int64 -> ``(slot [b*t, k], tok [E*b*cap])``."""
    n, k = idx.shape
    idx = _c(idx)
    slot = torch.empty(n, k, dtype=torch.int64, device=idx.device)
    tok = torch.empty(n_exp * b * cap, dtype=torch.int64, device=idx.device)
    L.call("bones_moe_slots", L.ptr(idx), L.ptr(slot), L.ptr(tok), _I(b), _I(t), _I(k), _I(n_exp), _I(cap), L.stream())
    COUNTS["moe_slots"] += 1
    return slot, tok


class _DispatchFn(torch.autograd.Function):
    """Forward: slot gather.  Backward: every token sums the gradients of its (at most k) slots -- the combine kernel
    with unit gates -- so both directions are gathers (reference: ``MoeGatherRows``, round2/source/train.py:10637)."""

    @staticmethod
    def forward(ctx, h, tok, slot):
        out = torch.empty(tok.numel(), h.shape[1], dtype=h.dtype, device=h.device)
        L.call("bones_gather_rows", L.ptr(h), L.ptr(tok), _I(1), L.ptr(out), _I(tok.numel()), _I(h.shape[1]),
               _L(h.shape[0]), L.stream())
        ctx.save_for_backward(tok, slot if slot is not None else tok)
        ctx.n, ctx.has_slot = h.shape[0], slot is not None
        COUNTS["moe_dispatch"] += 1
        return out

    @staticmethod
    def backward(ctx, dxs):
        tok, slot = ctx.saved_tensors
        dxs = _c(dxs)
        if ctx.has_slot:
            ones = torch.ones(slot.shape, dtype=torch.float32, device=dxs.device)
            dh = torch.empty(ctx.n, dxs.shape[1], dtype=dxs.dtype, device=dxs.device)
            L.call("bones_moe_combine", L.ptr(dxs), L.ptr(slot), L.ptr(ones), L.ptr(dh), _I(ctx.n), _I(dxs.shape[1]),
                   _I(slot.shape[1]), _L(dxs.shape[0]), L.stream())
            return dh, None, None
        g = torch.zeros(ctx.n, dxs.shape[1], dtype=torch.float32, device=dxs.device)
        L.call("bones_scatter_add_rows", L.ptr(dxs), L.ptr(tok), _I(1), L.ptr(g), _I(tok.numel()), _I(dxs.shape[1]),
               _L(ctx.n), L.stream())
        return g.to(dxs.dtype), None, None


def moe_dispatch(h, tok, slot=None):
    return _DispatchFn.apply(_c(h), _c(tok), _c(slot) if slot is not None else None)


class _CombineFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, ys, slot, gates):
        n, k = slot.shape
        out = torch.empty(n, ys.shape[1], dtype=ys.dtype, device=ys.device)
        g32 = _c(gates.float())
        L.call("bones_moe_combine", L.ptr(ys), L.ptr(slot), L.ptr(g32), L.ptr(out), _I(n), _I(ys.shape[1]), _I(k),
               _L(ys.shape[0]), L.stream())
        ctx.save_for_backward(ys, slot, g32)
        COUNTS["moe_combine"] += 1
        return out

    @staticmethod
    def backward(ctx, dout):
        ys, slot, g32 = ctx.saved_tensors
        dout = _c(dout)
        dys = torch.zeros_like(ys)
        dg = torch.empty_like(g32)
        L.call("bones_moe_combine_bwd", L.ptr(ys), L.ptr(slot), L.ptr(g32), L.ptr(dout), L.ptr(dys), L.ptr(dg), _I(slot.shape[0]),
               _I(ys.shape[1]), _I(slot.shape[1]), _L(ys.shape[0]), L.stream())
        return dys, None, dg


def moe_combine(ys, slot, gates):
    return _CombineFn.apply(_c(ys), _c(slot), gates)


class _ExpertsFn(torch.autograd.Function):
    """Local experts as one batched GEMM pair over ``[E_local, rows, d]`` (grouped by expert)."""

    @staticmethod
    def forward(ctx, xs, w_fc, w_proj):
        e, hdim, d = w_fc.shape
        x3 = _c(xs).view(e, -1, d)
        rows = x3.shape[1]
        h = torch.empty(e, rows, hdim, dtype=BF16, device=xs.device)
        L.gemm(x3, w_fc, h, m=rows, n=hdim, k=d, lda=d, ldb=d, ldd=hdim, epi=L.EPI_RELU2, batch=e, stride_a=rows * d,
               stride_b=hdim * d, stride_d=rows * hdim)
        y = torch.empty(e, rows, d, dtype=BF16, device=xs.device)
        L.gemm(h, w_proj, y, m=rows, n=d, k=hdim, lda=hdim, ldb=hdim, ldd=d, batch=e, stride_a=rows * hdim,
               stride_b=d * hdim, stride_d=rows * d)
        ctx.save_for_backward(x3, h, w_fc, w_proj)
        ctx.ws = (w_fc, w_proj)
        COUNTS["moe_experts"] += 1
        return y.view(xs.shape)

    @staticmethod
    def backward(ctx, dy):
        x3, h, w_fc, w_proj = ctx.saved_tensors
        e, hdim, d = w_fc.shape
        rows = x3.shape[1]
        dy3 = _c(dy).view(e, rows, d)
        dpre = torch.empty(e, rows, hdim, dtype=BF16, device=dy.device)
        L.gemm(dy3, w_proj, dpre, m=rows, n=hdim, k=d, lda=d, ldb=hdim, ldd=hdim, b_major=1, epi=L.EPI_MUL_2SQRT, r=h,
               ldr=hdim, batch=e, stride_a=rows * d, stride_b=d * hdim, stride_d=rows * hdim, stride_r=rows * hdim)
        dx = torch.empty(e, rows, d, dtype=BF16, device=dy.device)
        L.gemm(dpre, w_fc, dx, m=rows, n=d, k=hdim, lda=hdim, ldb=d, ldd=d, b_major=1, batch=e, stride_a=rows * hdim,
               stride_b=hdim * d, stride_d=rows * d)
        outs = []
        for w, a, b in ((ctx.ws[0], dpre, x3), (ctx.ws[1], dy3, h)):
            g = getattr(w, "main_grad", None)
            ret = None
            if g is None:
                g = ret = torch.zeros(w.shape, dtype=torch.float32, device=w.device)
            n_out, n_in = w.shape[1], w.shape[2]
            L.gemm(a, b, g, m=n_out, n=n_in, k=rows, lda=n_out, ldb=n_in, ldd=n_in, a_major=1, b_major=1,
                   epi=L.EPI_ACC_F32, batch=e, stride_a=rows * n_out, stride_b=rows * n_in, stride_d=n_out * n_in)
            outs.append(ret.to(w.dtype) if ret is not None else None)
        COUNTS["gemm"] += 4
        return dx.view(dy.shape), outs[0], outs[1]


def moe_experts(xs, w_fc, w_proj, precision="bf16"):
    if precision == "mxfp8":
        from . import mxfp8
        if mxfp8.experts_apply(xs, w_fc, w_proj):
            return mxfp8._MxExpertsFn.apply(xs, w_fc, w_proj)
    return _ExpertsFn.apply(xs, w_fc, w_proj)


# -- tables ----------------------------------------------------------------------------------------------------------
def sparse_adam_rows(table, rows, g, m, v, step, lr, beta1, beta2, eps, decay):
    if table.dtype != BF16:
        raise RuntimeError("native sparse Adam expects a bf16 table")
    L.call("bones_sparse_adam", L.ptr(table), L.ptr(_c(rows)), L.ptr(_c(g)), L.ptr(m), L.ptr(v), _I(rows.numel()),
           _I(table.shape[1]), _F(lr), _F(beta1), _F(beta2), _F(eps), _F(decay), _I(step), L.stream())
    COUNTS["sparse_adam"] += 1
