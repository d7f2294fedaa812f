"""Autograd wrapper of the sm_100a attention kernels (``csrc/attention.cu``, ``csrc/attention_bwd_split.cu``).

Forward: RoPE + QK-norm pre-pass into a ``[B*T, 2*H*D]`` buffer, then the persistent tcgen05 flash-attention kernel
reading the values in place from the packed ``qkv``.  Saved for backward: ``qkv``, the rotated/normalised ``qk``, the
output and ``lse``.  Backward (``ops/attention_bwd.py``): a statistics pre-pass, the dK/dV kernel and the dQ kernel
(every accumulator in TMEM, bf16 outputs, no atomics), then the pre-pass backward that applies the norm Jacobian and
the inverse rotation and writes one packed ``[B, T, 3*H*D]`` gradient (reference: the fused backward emits one packed
gradient, round2/source/kernels/nki_attn_bandpro.py:1-134).
"""
from __future__ import annotations

import ctypes

import torch

from . import _lib as L

_I, _L, _F = ctypes.c_int, ctypes.c_longlong, ctypes.c_float
SUPPORTED_HEAD_DIMS = (128, 64)        # 64: zero-padded to the kernels' 128 (see _AttnPad64Fn)


def why_not(qkv, n_head, head_dim, window=0) -> str:
    """Empty when the kernels cover the call, else the reason."""
    if qkv.dtype != torch.bfloat16:
        return f"dtype {qkv.dtype} (bf16 only)"
    if head_dim not in SUPPORTED_HEAD_DIMS:
        return f"head_dim {head_dim} (supported: {SUPPORTED_HEAD_DIMS})"
    if qkv.shape[1] % 128:
        return f"sequence length {qkv.shape[1]} is not a multiple of 128"
    if window % 128:
        return f"window {window} is not a multiple of 128"
    return ""


def applies(qkv, n_head, head_dim) -> bool:
    return not why_not(qkv, n_head, head_dim)


def rope_qknorm(qkv2, cos, sin, t, n_head, head_dim):
    m = qkv2.shape[0]
    qk = torch.empty(m, 2 * n_head * head_dim, dtype=qkv2.dtype, device=qkv2.device)
    L.call("bones_rope_qknorm_fwd", L.ptr(qkv2), L.ptr(cos), L.ptr(sin), L.ptr(qk), _L(m), _I(t), _I(n_head), _I(head_dim),
           L.stream())
    return qk


def attn_forward(qk, qkv2, doc_start, b, t, n_head, scale, window):
    y = torch.empty(b * t, n_head * 128, dtype=qkv2.dtype, device=qkv2.device)
    lse = torch.empty(b, n_head, t, dtype=torch.float32, device=qkv2.device)
    L.call("bones_attn_fwd", L.ptr(qk), L.ptr(qkv2), L.ptr(y), L.ptr(lse), L.ptr(doc_start), _I(b), _I(t), _I(n_head), _F(scale),
           _I(window // 128), L.stream())
    return y, lse


class _AttnFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, qkv, cos, sin, n_head, head_dim, scale, doc_start, window):
        b, t, _ = qkv.shape
        qkv2 = (qkv if qkv.is_contiguous() else qkv.contiguous()).view(b * t, -1)
        cos, sin = cos.float().contiguous(), sin.float().contiguous()
        ds = doc_start.to(torch.int32).contiguous() if doc_start is not None else None
        qk = rope_qknorm(qkv2, cos, sin, t, n_head, head_dim)
        y, lse = attn_forward(qk, qkv2, ds, b, t, n_head, scale, window)
        ctx.save_for_backward(qkv2, qk, y, lse, cos, sin, ds)
        ctx.meta = (b, t, n_head, head_dim, scale, window)
        return y.view(b, t, n_head * head_dim)

    @staticmethod
    def backward(ctx, dy):
        qkv2, qk, y, lse, cos, sin, ds = ctx.saved_tensors
        b, t, n_head, head_dim, scale, window = ctx.meta
        from . import attention_bwd as AB
        dqkv = AB.backward(dy, qkv2, qk, y, lse, cos, sin, ds, b, t, n_head, head_dim, scale, window)
        return dqkv.view(b, t, -1), None, None, None, None, None, None, None


class _AttnPad64Fn(torch.autograd.Function):
    """head_dim 64 on the head_dim-128 kernels.  RoPE and the QK-norm run on the real 64 dimensions (their kernels are
    templated on the head dim); the rotated, normalised q and k and the values are then laid out as 128-wide heads whose
    upper halves are zero, which changes neither ``q . k`` nor the lower half of ``P V``.  The tensor-core kernels do
    twice the work a native 64-wide kernel would, which is the price of not having one: the tiny configurations that
    use this head width are not the ones the kernels were sized for.  (The softmax's fixed shift ``scale * 128`` is
    above the largest possible logit ``scale * 64``, so it stays valid.)"""

    @staticmethod
    def _pad(x2, heads):              # [M, heads * 64] -> [M, heads * 128], upper half of every head zero
        m = x2.shape[0]
        out = torch.zeros(m, heads, 128, dtype=x2.dtype, device=x2.device)
        out[:, :, :64] = x2.view(m, heads, 64)
        return out.view(m, heads * 128)

    @staticmethod
    def forward(ctx, qkv, cos, sin, n_head, scale, doc_start, window):
        b, t, _ = qkv.shape
        a = n_head * 64
        qkv2 = (qkv if qkv.is_contiguous() else qkv.contiguous()).view(b * t, 3 * a)
        cos, sin = cos.float().contiguous(), sin.float().contiguous()
        ds = doc_start.to(torch.int32).contiguous() if doc_start is not None else None
        qk = rope_qknorm(qkv2, cos, sin, t, n_head, 64)
        qkp = _AttnPad64Fn._pad(qk, 2 * n_head)
        # the kernels read the values at column 2 * A' of rows 3 * A' wide: a packed buffer whose q and k thirds stay unused
        qkvp = torch.zeros(b * t, 3 * n_head * 128, dtype=qkv2.dtype, device=qkv2.device)
        qkvp[:, 2 * n_head * 128:] = _AttnPad64Fn._pad(qkv2[:, 2 * a:], n_head)
        y128, lse = attn_forward(qkp, qkvp, ds, b, t, n_head, scale, window)
        ctx.save_for_backward(qkv2, qkp, qkvp, y128, lse, cos, sin, ds)
        ctx.meta = (b, t, n_head, scale, window)
        return y128.view(b * t, n_head, 128)[:, :, :64].reshape(b, t, a)

    @staticmethod
    def backward(ctx, dy):
        qkv2, qkp, qkvp, y128, lse, cos, sin, ds = ctx.saved_tensors
        b, t, n_head, scale, window = ctx.meta
        m, a, ap = b * t, n_head * 64, n_head * 128
        dev = dy.device
        dy128 = _AttnPad64Fn._pad((dy if dy.is_contiguous() else dy.contiguous()).view(m, a), n_head)
        stats = torch.empty(b, n_head, t, 2, dtype=torch.float32, device=dev)
        L.call("bones_attn_bwd_stats", L.ptr(dy128), L.ptr(y128), L.ptr(lse), L.ptr(stats), _L(m), _I(t), _I(n_head), L.stream())
        dqk128 = torch.empty(m, 2 * ap, dtype=torch.bfloat16, device=dev)
        dv128 = torch.empty(m, ap, dtype=torch.bfloat16, device=dev)
        L.call("bones_attn_bwd_split", L.ptr(qkp), L.ptr(qkvp), L.ptr(dy128), L.ptr(stats), L.ptr(dqk128), L.ptr(dv128), _L(ap), L.ptr(ds),
               _I(b), _I(t), _I(n_head), _F(scale), _I(window // 128), L.stream())
        dqk = dqk128.view(m, 2 * n_head, 128)[:, :, :64].float().reshape(m, 2 * a).contiguous()
        dv = dv128.view(m, n_head, 128)[:, :, :64].reshape(m, a).contiguous()
        dqkv = torch.empty(m, 3 * a, dtype=torch.bfloat16, device=dev)
        L.call("bones_rope_qknorm_bwd", L.ptr(qkv2), L.ptr(cos), L.ptr(sin), L.ptr(dqk), L.ptr(dv), L.ptr(dqkv), _L(m), _I(t), _I(n_head),
               _I(64), L.stream())
        return dqkv.view(b, t, 3 * a), None, None, None, None, None, None


def attention(qkv, cos, sin, n_head, head_dim, scale, doc_start, window):
    if head_dim == 64:
        return _AttnPad64Fn.apply(qkv, cos, sin, n_head, scale, doc_start, window)
    return _AttnFn.apply(qkv, cos, sin, n_head, head_dim, scale, doc_start, window)
