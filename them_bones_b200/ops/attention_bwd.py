"""Backward of the native attention: delta pre-pass, tcgen05 backward kernel, RoPE/QK-norm backward."""
from __future__ import annotations

import ctypes
import os

import torch

from . import _lib as L

_I, _L, _F = ctypes.c_int, ctypes.c_longlong, ctypes.c_float
# split: two kernels (dK/dV, then dQ), every accumulator in TMEM; fused: one kernel with dQ through fp32 atomics
_IMPL = os.environ.get("BONES_ATTN_BWD", "split")


def backward(dy, qkv2, qk, y, lse, cos, sin, ds, b, t, n_head, head_dim, scale, window):
    m, a = b * t, n_head * head_dim
    dy2 = (dy if dy.is_contiguous() else dy.contiguous()).view(m, a)
    delta = torch.empty(b, n_head, t, dtype=torch.float32, device=dy.device)
    L.call("bones_attn_delta", L.ptr(dy2), L.ptr(y), L.ptr(delta), _L(m), _I(t), _I(n_head), L.stream())
    dqk = torch.empty(m, 2 * a, dtype=torch.float32, device=dy.device)
    dv = torch.empty(m, a, dtype=torch.bfloat16, device=dy.device)
    L.call("bones_attn_bwd" if _IMPL == "fused" else "bones_attn_bwd_split", L.ptr(qk), L.ptr(qkv2), L.ptr(dy2), L.ptr(lse), L.ptr(delta), L.ptr(dqk), L.ptr(dv), L.ptr(ds),
           _I(b), _I(t), _I(n_head), _F(scale), _I(window // 128), L.stream())
    dqkv = torch.empty(m, 3 * a, dtype=torch.bfloat16, device=dy.device)
    L.call("bones_rope_qknorm_bwd", L.ptr(qkv2), L.ptr(cos), L.ptr(sin), L.ptr(dqk), L.ptr(dv), L.ptr(dqkv), _L(m), _I(t),
           _I(n_head), _I(head_dim), L.stream())
    return dqkv
