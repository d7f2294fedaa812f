"""``torch.library`` registration of the native kernels: custom ops with fake (shape-only) implementations and autograd
formulas, so the kernels are visible to ``torch.compile`` / ``torch.export`` / fake-tensor tracing as ordinary ops in the
``bones::`` namespace instead of opaque Python calls.

Reference: ``register_attn_ops`` (round2/source/train.py:4964-5042) registers each kernel as a ``custom_op`` with a
``register_fake`` shape function and a ``register_autograd`` pair whose ``setup_context`` saves tensors and marks the
auxiliary outputs (statistics kept for backward) non-differentiable; the same structure is used here.

Registered ops (each runs the same C entry point as the eager wrappers in ``ops/cuda.py`` / ``ops/attention_native.py``):

* ``bones::attention_fwd(qkv, cos, sin, doc_start?, n_head, head_dim, scale, window) -> (y, lse, qk)`` and
  ``bones::attention_bwd(dy, qkv, qk, y, lse, cos, sin, doc_start?, ...) -> dqkv``
* ``bones::rmsnorm_fwd(x) -> y`` and ``bones::rmsnorm_bwd(x, dy) -> dx``

``attention`` / ``rms_norm`` below are the differentiable entry points.  ``BONES_LIBRARY_OPS=1`` routes the model's
attention and norms through them (the default eager wrappers skip the dispatcher's per-call cost).
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch
from torch import Tensor

_LIB = "bones"


# -- attention --------------------------------------------------------------------------------------------------------
@torch.library.custom_op(f"{_LIB}::attention_fwd", mutates_args=())
def attention_fwd(qkv: Tensor, cos: Tensor, sin: Tensor, doc_start: Optional[Tensor], n_head: int, head_dim: int, scale: float,
                  window: int) -> Tuple[Tensor, Tensor, Tensor]:
    from . import attention_native as AN
    b, t, _ = qkv.shape
    qkv2 = qkv.contiguous().view(b * t, -1)
    qk = AN.rope_qknorm(qkv2, cos, sin, t, n_head, head_dim)
    y, lse = AN.attn_forward(qk, qkv2, doc_start, b, t, n_head, scale, window)
    return y.view(b, t, n_head * head_dim), lse, qk


@attention_fwd.register_fake
def _(qkv, cos, sin, doc_start, n_head, head_dim, scale, window):
    b, t, _ = qkv.shape
    a = n_head * head_dim
    return (qkv.new_empty(b, t, a), qkv.new_empty(b, n_head, t, dtype=torch.float32), qkv.new_empty(b * t, 2 * a))


@torch.library.custom_op(f"{_LIB}::attention_bwd", mutates_args=())
def attention_bwd(dy: Tensor, qkv: Tensor, qk: Tensor, y: Tensor, lse: Tensor, cos: Tensor, sin: Tensor, doc_start: Optional[Tensor],
                  n_head: int, head_dim: int, scale: float, window: int) -> Tensor:
    from . import attention_bwd as AB
    b, t, _ = qkv.shape
    qkv2 = qkv.contiguous().view(b * t, -1)
    dqkv = AB.backward(dy, qkv2, qk, y.reshape(b * t, -1), lse, cos, sin, doc_start, b, t, n_head, head_dim, scale, window)
    return dqkv.view(b, t, -1)


@attention_bwd.register_fake
def _(dy, qkv, qk, y, lse, cos, sin, doc_start, n_head, head_dim, scale, window):
    return torch.empty_like(qkv)


def _attn_setup(ctx, inputs, output):
    qkv, cos, sin, doc_start, n_head, head_dim, scale, window = inputs
    y, lse, qk = output
    ctx.save_for_backward(qkv, qk, y, lse, cos, sin, doc_start)
    ctx.meta = (n_head, head_dim, scale, window)
    ctx.mark_non_differentiable(lse, qk)             # statistics and the rotated copy exist for backward only


def _attn_backward(ctx, dy, _dlse, _dqk):
    qkv, qk, y, lse, cos, sin, doc_start = ctx.saved_tensors
    n_head, head_dim, scale, window = ctx.meta
    dqkv = torch.ops.bones.attention_bwd(dy.contiguous(), qkv, qk, y, lse, cos, sin, doc_start, n_head, head_dim, scale, window)
    return dqkv, None, None, None, None, None, None, None


attention_fwd.register_autograd(_attn_backward, setup_context=_attn_setup)


def attention(qkv, cos, sin, n_head, head_dim, scale, doc_start=None, window=0):
    ds = doc_start.to(torch.int32).contiguous() if doc_start is not None else None
    y, _, _ = torch.ops.bones.attention_fwd(qkv, cos.float().contiguous(), sin.float().contiguous(), ds, n_head, head_dim,
                                            float(scale), int(window))
    return y


# -- RMSNorm ------------------------------------------------------------------------------------------------------------
@torch.library.custom_op(f"{_LIB}::rmsnorm_fwd", mutates_args=())
def rmsnorm_fwd(x: Tensor) -> Tensor:
    import ctypes

    from . import _lib as L
    x2 = x.contiguous().view(-1, x.shape[-1])
    y = torch.empty_like(x2)
    L.call("bones_rmsnorm_fwd", L.ptr(x2), L.ptr(y), ctypes.c_int(x2.shape[0]), ctypes.c_int(x2.shape[1]), L.stream())
    return y.view(x.shape)


@rmsnorm_fwd.register_fake
def _(x):
    return torch.empty_like(x)


@torch.library.custom_op(f"{_LIB}::rmsnorm_bwd", mutates_args=())
def rmsnorm_bwd(x: Tensor, dy: Tensor) -> Tensor:
    import ctypes

    from . import _lib as L
    x2 = x.contiguous().view(-1, x.shape[-1])
    dy2 = dy.contiguous().view(x2.shape)
    dx = torch.empty_like(x2)
    L.call("bones_rmsnorm_bwd", L.ptr(x2), L.ptr(dy2), L.ptr(None), L.ptr(dx), ctypes.c_int(x2.shape[0]), ctypes.c_int(x2.shape[1]),
           L.stream())
    return dx.view(x.shape)


@rmsnorm_bwd.register_fake
def _(x, dy):
    return torch.empty_like(x)


def _rms_setup(ctx, inputs, output):
    ctx.save_for_backward(inputs[0])


def _rms_backward(ctx, dy):
    (x,) = ctx.saved_tensors
    return torch.ops.bones.rmsnorm_bwd(x, dy)


rmsnorm_fwd.register_autograd(_rms_backward, setup_context=_rms_setup)


def rms_norm(x):
    return torch.ops.bones.rmsnorm_fwd(x)


OPS = ("attention_fwd", "attention_bwd", "rmsnorm_fwd", "rmsnorm_bwd")
