"""Backward of the native attention: statistics pre-pass, tcgen05 backward kernels, RoPE/QK-norm backward."""
from __future__ import annotations

import ctypes
import os

import torch

from . import _lib as L

_I, _L, _F = ctypes.c_int, ctypes.c_longlong, ctypes.c_float
# split: two kernels (dK/dV, then dQ), every accumulator and every intermediate in TMEM, bf16 outputs;
# fused: one kernel with dQ through fp32 atomics
_IMPL = os.environ.get("BONES_ATTN_BWD", "split")


def backward(dy, qkv2, qk, y, lse, cos, sin, ds, b, t, n_head, head_dim, scale, window):
    m, a = b * t, n_head * head_dim
    dev = dy.device
    dy2 = (dy if dy.is_contiguous() else dy.contiguous()).view(m, a)
    dqkv = torch.empty(m, 3 * a, dtype=torch.bfloat16, device=dev)
    if _IMPL != "fused" and head_dim == 128:
        stats = torch.empty(b, n_head, t, 2, dtype=torch.float32, device=dev)
        L.call("bones_attn_bwd_stats", L.ptr(dy2), L.ptr(y), L.ptr(lse), L.ptr(stats), _L(m), _I(t), _I(n_head), L.stream())
        dqk = torch.empty(m, 2 * a, dtype=torch.bfloat16, device=dev)
        dv = dqkv[:, 2 * a:]                                   # the kernel writes dV in place, rows 3a apart
        L.call("bones_attn_bwd_split", L.ptr(qk), L.ptr(qkv2), L.ptr(dy2), L.ptr(stats), L.ptr(dqk), L.ptr(dv), _L(3 * a), L.ptr(ds),
               _I(b), _I(t), _I(n_head), _F(scale), _I(window // 128), L.stream())
        L.call("bones_rope_qknorm_bwd_bf16", L.ptr(qkv2), L.ptr(cos), L.ptr(sin), L.ptr(dqk), L.ptr(dqkv), _L(m), _I(t), _I(n_head),
               L.stream())
        return dqkv
    delta = torch.empty(b, n_head, t, dtype=torch.float32, device=dev)
    L.call("bones_attn_delta", L.ptr(dy2), L.ptr(y), L.ptr(delta), _L(m), _I(t), _I(n_head), L.stream())
    dqk = torch.empty(m, 2 * a, dtype=torch.float32, device=dev)
    dv = torch.empty(m, a, dtype=torch.bfloat16, device=dev)
    L.call("bones_attn_bwd", L.ptr(qk), L.ptr(qkv2), L.ptr(dy2), L.ptr(lse), L.ptr(delta), L.ptr(dqk), L.ptr(dv), L.ptr(ds),
           _I(b), _I(t), _I(n_head), _F(scale), _I(window // 128), L.stream())
    L.call("bones_rope_qknorm_bwd", L.ptr(qkv2), L.ptr(cos), L.ptr(sin), L.ptr(dqk), L.ptr(dv), L.ptr(dqkv), _L(m), _I(t),
           _I(n_head), _I(head_dim), L.stream())
    return dqkv
