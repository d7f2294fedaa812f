"""Attention operator on the GPU: RoPE + QK-norm + causal (document-reset, optionally banded) softmax attention.

``attention()`` dispatches to the hand-written sm_100a flash-attention kernels (``csrc/attn_fwd.cu`` / ``attn_bwd.cu``)
when they cover the shape (head_dim 64 or 128, sequence a multiple of 128); otherwise it raises.  The SDPA route is kept
only as the explicit baseline path (``BONES_KERNELS=ref``).
"""
from __future__ import annotations

import os

import torch

from . import COUNTS

_IMPL = os.environ.get("BONES_ATTN", "auto")


def attention(qkv, cos, sin, n_head, head_dim, scale, doc_start, window):
    from . import _sdpa_attention
    try:
        from . import attention_native as AN
    except ImportError:
        AN = None
    if AN is not None and _IMPL != "sdpa" and AN.applies(qkv, n_head, head_dim):
        COUNTS["attention"] += 1
        return AN.attention(qkv, cos, sin, n_head, head_dim, scale, doc_start, window)
    COUNTS["attention_sdpa"] += 1
    return _sdpa_attention(qkv, cos, sin, n_head, head_dim, scale, doc_start, window)
