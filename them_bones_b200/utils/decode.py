"""Greedy decoding with a KV cache.

The reference scores teacher-forced full sequences only (round2/submission/inference.py:26-27); autoregressive decoding
is an added capability.  The cache stores, per layer, keys *after* RoPE and QK-norm and raw values, so a decode step
rotates only the new token (RoPE at its absolute position) and attends over the cached prefix restricted to the current
document and the layer's window.
"""
from __future__ import annotations

import torch
import torch.nn.functional as F

from .. import ops
from ..models.moe import MoeMLP
from ..ref import functional as RF


class KVCache:
    def __init__(self, model, batch: int, max_len: int):
        cfg = model.config
        dev, dt = model.lm_head.weight.device, model.lm_head.weight.dtype
        shape = (cfg.n_layer, batch, max_len, cfg.n_head, cfg.head_dim)
        self.k = torch.zeros(shape, dtype=dt, device=dev)
        self.v = torch.zeros(shape, dtype=dt, device=dev)
        self.doc_start = torch.zeros(batch, dtype=torch.int32, device=dev)
        self.len = 0


def _attend(q, k, v, scale, lo):
    """q ``[B,H,1,D]``, k/v ``[B,L,H,D]``; keys at positions < ``lo[b]`` are masked."""
    b, l = k.shape[0], k.shape[1]
    s = torch.einsum("bhqd,blhd->bhql", q.float(), k.float()) * scale
    pos = torch.arange(l, device=k.device)[None, None, None, :]
    s = s.masked_fill(pos < lo[:, None, None, None], float("-inf"))
    return torch.einsum("bhql,blhd->bqhd", torch.softmax(s, -1), v.float())


@torch.no_grad()
def _forward_cached(model, idx, cache: KVCache):
    """Run ``idx [B, t]`` (the whole prompt at prefill, one token afterwards), appending to the cache.  Returns the
    logits of the last position ``[B, V]``."""
    cfg = model.config
    b, t = idx.shape
    p0 = cache.len
    dev = idx.device
    pos = torch.arange(p0, p0 + t, device=dev)
    # document starts: most recent BOS at or before each new position
    if cfg.doc_mask:
        marks = torch.where(idx == cfg.bos_id, pos[None, :].expand(b, t).to(torch.int32),
                            torch.zeros(b, t, dtype=torch.int32, device=dev))
        ds = torch.maximum(torch.cummax(marks, 1).values, cache.doc_start[:, None])
        cache.doc_start = ds[:, -1].clone()
    else:
        ds = torch.zeros(b, t, dtype=torch.int32, device=dev)
    cos, sin = model.cos[p0:p0 + t], model.sin[p0:p0 + t]
    x = F.embedding(idx, model.transformer.wte.weight)
    if model.tables is not None:
        raise NotImplementedError("cached decoding with hashed tables goes through decode_with_tables")
    x = RF.rms_norm(x)
    x0 = x
    skips = []
    n_layer, n_skip = cfg.n_layer, model.n_skip
    for i, blk in enumerate(model.transformer.h):
        if n_skip and i >= n_layer - n_skip:
            x = x + model.skip_lambda[i - (n_layer - n_skip)].to(x.dtype) * skips.pop()
        x = RF.resid_mix(x, x0, blk.resid_lambda, blk.x0_lambda)
        xn = RF.rms_norm(x)
        at = blk.attn
        q = F.linear(xn, at.c_q.weight).view(b, t, at.n_head, at.head_dim)
        k = F.linear(xn, at.c_k.weight).view(b, t, at.n_head, at.head_dim)
        v = F.linear(xn, at.c_v.weight).view(b, t, at.n_head, at.head_dim)
        if model.value_embeds is not None and str(i) in model.value_embeds:
            ve = F.embedding(idx, model.value_embeds[str(i)].weight).view(b, t, at.n_head, at.head_dim)
            v = v + blk.ve_lambda.to(v.dtype) * ve.to(v.dtype)
        q = RF.rms_norm(_rope_at(q, cos, sin))
        k = RF.rms_norm(_rope_at(k, cos, sin))
        cache.k[i, :, p0:p0 + t] = k
        cache.v[i, :, p0:p0 + t] = v
        ys = []
        for j in range(t):                                   # prefill is short in decode benchmarks; one row at a time
            cur = p0 + j
            lo = ds[:, j].to(torch.int64)
            if at.window:
                lo = torch.maximum(lo, torch.full_like(lo, max(0, (cur // 128 - (at.window // 128 - 1)) * 128)))
            ys.append(_attend(q[:, j:j + 1].transpose(1, 2), cache.k[i, :, :cur + 1], cache.v[i, :, :cur + 1],
                              at.scale, lo))
        y = torch.cat(ys, 1).reshape(b, t, -1).to(x.dtype)
        x = x + F.linear(y, at.c_proj.weight)
        xn = RF.rms_norm(x)
        if isinstance(blk.mlp, MoeMLP):
            x = blk.mlp(xn, residual=x)
        else:
            x = x + RF.mlp(xn, blk.mlp.c_fc.weight, blk.mlp.c_proj.weight)
        if n_skip and i < n_skip:
            skips.append(x)
    cache.len = p0 + t
    x = RF.rms_norm(x[:, -1])
    return RF.softcap_logits(F.linear(x, model.lm_head.weight)[..., :cfg.vocab_size], cfg.softcap)


def _rope_at(x, cos, sin):
    d = x.shape[-1] // 2
    x1, x2 = x[..., :d].float(), x[..., d:].float()
    c, s = cos[None, :, None, :].float(), sin[None, :, None, :].float()
    return torch.cat([x1 * c + x2 * s, -x1 * s + x2 * c], -1).to(x.dtype)


@torch.no_grad()
def greedy_decode(model, prompts: torch.Tensor, n_new: int) -> torch.Tensor:
    """``prompts [B, P]`` -> ``[B, P + n_new]`` by arg-max decoding."""
    b, p = prompts.shape
    if p + n_new > model.config.sequence_len:
        raise ValueError("prompt + new tokens exceed the model's sequence length")
    if model.tables is not None:
        return greedy_decode_full(model, prompts, n_new)
    cache = KVCache(model, b, p + n_new)
    out = [prompts]
    logits = _forward_cached(model, prompts, cache)
    for _ in range(n_new):
        nxt = logits.argmax(-1, keepdim=True)
        out.append(nxt)
        if cache.len >= p + n_new:
            break
        logits = _forward_cached(model, nxt, cache)
    return torch.cat(out, 1)[:, :p + n_new]


@torch.no_grad()
def greedy_decode_full(model, prompts: torch.Tensor, n_new: int) -> torch.Tensor:
    """Cache-free decoding (re-runs the full forward per token); the oracle for the cached path and the route used
    when hashed tables are attached."""
    seq = prompts
    for _ in range(n_new):
        logits = model(seq)[:, -1]
        seq = torch.cat([seq, logits.argmax(-1, keepdim=True)], 1)
    return seq
