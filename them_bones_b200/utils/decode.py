"""Greedy decoding with a KV cache.

The reference scores teacher-forced full sequences only (round2/submission/inference.py:26-27); autoregressive decoding
is an added capability.  The cache stores, per layer, keys *after* RoPE and QK-norm and raw values, so a decode step
rotates only the new token (RoPE at its absolute position) and attends over the cached prefix restricted to the current
document and the layer's window.
"""
from __future__ import annotations

import ctypes

import torch
import torch.nn.functional as F

from .. import ops
from ..models.moe import MoeMLP
from ..ref import functional as RF


def L_check():
    from ..ops import _lib as L
    L.check_error_word()


class KVCache:
    def __init__(self, model, batch: int, max_len: int):
        cfg = model.config
        dev, dt = model.lm_head.weight.device, model.lm_head.weight.dtype
        shape = (cfg.n_layer, batch, max_len, cfg.n_head, cfg.head_dim)
        self.k = torch.zeros(shape, dtype=dt, device=dev)
        self.v = torch.zeros(shape, dtype=dt, device=dev)
        self.doc_start = torch.zeros(batch, dtype=torch.int32, device=dev)
        self.len = 0
        self.tokens = None          # token history [batch, max_len], kept when the model has hashed tables


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
        # rows keyed by the last `order` tokens: the cache keeps the token history for contexts that start before this call
        if cache.tokens is None:
            cache.tokens = torch.zeros(b, cache.k.shape[2], dtype=torch.int64, device=dev)
        cache.tokens[:, p0:p0 + t] = idx
        hist, tb = cache.tokens[:, :p0 + t], model.tables
        ids = torch.stack([RF.ngram_rows(hist, o, tb.rows, tb.seed + j, _doc_start_full(hist, cfg) if cfg.doc_mask else None)[:, p0:]
                           for j, o in enumerate(tb.orders)])
        x = tb.add_lookup(x, idx, None, model.table_lambda, rows=ids)
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


def _doc_start_full(hist, cfg):
    return RF.doc_start_positions(hist, cfg.bos_id)


def _rope_at(x, cos, sin):
    d = x.shape[-1] // 2
    x1, x2 = x[..., :d].float(), x[..., d:].float()
    c, s = cos[None, :, None, :].float(), sin[None, :, None, :].float()
    return torch.cat([x1 * c + x2 * s, -x1 * s + x2 * c], -1).to(x.dtype)


class NativeDecoder:
    """One decode step as a CUDA graph over the native kernels: embedding, fused norms, tcgen05 GEMMs, the two decode
    kernels (``csrc/decode.cu``: RoPE + QK-norm + cache append, cached attention), soft-capped logits, arg-max.  The
    position, the per-sequence document starts, the current tokens and the output buffer live on the device and are
    advanced inside the graph, so generating ``n`` tokens is ``n`` graph replays with no host synchronisation.
    Eligible: bf16 models on CUDA whose blocks all have attention with head_dim 128.  MoE blocks run their routed experts
    inside the graph (router, slotting, grouped expert GEMMs, combine: all device-side, a decode step uses one slot per
    sequence and expert); hashed input tables are looked up from row ids hashed on the device from the token history."""

    @staticmethod
    def eligible(model) -> bool:
        cfg = model.config
        w = model.lm_head.weight
        tables_ok = model.tables is None or model.tables.dtype == torch.bfloat16
        return (w.is_cuda and w.dtype == torch.bfloat16 and cfg.head_dim == 128 and tables_ok and getattr(model, "os1", None) is None
                and not ops.reference_path() and all(blk.attn is not None for blk in model.transformer.h))

    def __init__(self, model, cache: KVCache, first_tokens: torch.Tensor, out: torch.Tensor, prompt_len: int = 0):
        # positions below ``prompt_len`` are teacher-forced from ``out`` (stepwise prefill through the same graph)
        self.model, self.cache, self.out = model, cache, out
        dev = first_tokens.device
        self.prompt_len = torch.tensor([prompt_len], dtype=torch.int32, device=dev)
        self.tok = first_tokens.clone().to(torch.int64)
        self.pos = torch.tensor([cache.len], dtype=torch.int32, device=dev)
        self.graph = None
        cfg = model.config
        b, a = self.tok.shape[0], cfg.n_head * cfg.head_dim
        self.qbuf = torch.empty(b, a, dtype=torch.bfloat16, device=dev)
        self.y = torch.empty(b, a, dtype=torch.bfloat16, device=dev)
        # With few rows a projection has too few output tiles to pull its weights at memory speed, so its contraction
        # runs as a batch of products over K chunks of 256, each into its own fp32 slice, which the finishing kernel
        # adds in a fixed order (no atomics: a step is reproducible bit for bit).
        self.split = b <= 128 and cfg.n_embd % 256 == 0 and a % 256 == 0
        self.dense = [not isinstance(blk.mlp, MoeMLP) for blk in model.transformer.h]
        if self.split:
            self.wqkv = [torch.cat([blk.attn.c_q.weight, blk.attn.c_k.weight, blk.attn.c_v.weight]).contiguous()
                         for blk in model.transformer.h]
            ws = self.wqkv + [blk.attn.c_proj.weight for blk in model.transformer.h]
            ws += [w for blk, dense in zip(model.transformer.h, self.dense) if dense for w in (blk.mlp.c_fc.weight, blk.mlp.c_proj.weight)]
            self.split = all(w.shape[1] % 256 == 0 for w in ws)
            self.part = torch.empty(max(b * w.shape[0] * (w.shape[1] // 256) for w in ws), dtype=torch.float32, device=dev)

    def _lin(self, x, w, mode=0, residual=None):
        """``x [b, k] @ w[n, k]^T`` as ``k / 256`` batched partial products into fp32 slices, then their ordered sum as
        bf16 (mode 0), through ReLU^2 (2) or ``+ residual`` (1)."""
        from ..ops import _lib as L
        b, k = x.shape
        n = w.shape[0]
        splits = k // 256
        part = self.part[:splits * b * n]
        L.gemm(x, w, part, m=b, n=n, k=256, lda=x.stride(0), ldb=w.stride(0), ldd=n, epi=L.EPI_F32, force_bn=128, pair=False,
               batch=splits, stride_a=256, stride_b=256, stride_d=b * n)
        out = torch.empty(b, n, dtype=torch.bfloat16, device=x.device)
        L.call("bones_acc_finish", L.ptr(part), ctypes.c_int(splits), ctypes.c_longlong(b * n), L.ptr(residual), L.ptr(out),
               ctypes.c_longlong(b * n), ctypes.c_int(mode), L.stream())
        return out

    def _step(self):
        from ..ops import _lib as L
        from ..ops import cuda as C
        model, cache, cfg = self.model, self.cache, self.model.config
        tok, pos = self.tok, self.pos
        b, tmax = tok.shape[0], cache.k.shape[2]
        if cfg.doc_mask:
            cache.doc_start.copy_(torch.where(tok == cfg.bos_id, pos.expand(b), cache.doc_start))
        x = ops.embedding(tok, model.transformer.wte.weight, torch.bfloat16)
        if model.tables is not None:
            tb = model.tables
            ds = cache.doc_start if cfg.doc_mask else None
            for j, o in enumerate(tb.orders):
                rows = RF.ngram_rows_at(self.out, pos, o, tb.rows, tb.seed + j, ds)
                x = x + model.table_lambda[j].to(x.dtype) * tb.gather(j, rows)
        x = ops.rms_norm(x)
        x0 = x
        skips = []
        n_layer, n_skip = cfg.n_layer, model.n_skip
        for i, blk in enumerate(model.transformer.h):
            if n_skip and i >= n_layer - n_skip:
                x = x + model.skip_lambda[i - (n_layer - n_skip)].to(x.dtype) * skips.pop()
            x, xn = ops.resid_mix_norm(x, x0, blk.resid_lambda, blk.x0_lambda)
            at = blk.attn
            qkv = self._lin(xn, self.wqkv[i]) if self.split else ops.linear_qkv(xn, at.c_q.weight, at.c_k.weight, at.c_v.weight)
            ve = lam = None
            if model.value_embeds is not None and str(i) in model.value_embeds:
                ve = ops.embedding(tok, model.value_embeds[str(i)].weight, torch.bfloat16)
                lam = blk.ve_lambda.detach().float()
            L.call("bones_decode_qkv", L.ptr(qkv), L.ptr(model.cos), L.ptr(model.sin), L.ptr(ve), L.ptr(lam), L.ptr(self.qbuf),
                   L.ptr(cache.k[i]), L.ptr(cache.v[i]), L.ptr(pos), C._I(b), C._I(at.n_head), C._I(tmax), L.stream())
            L.call("bones_decode_attn", L.ptr(self.qbuf), L.ptr(cache.k[i]), L.ptr(cache.v[i]), L.ptr(pos),
                   L.ptr(cache.doc_start if cfg.doc_mask else None), L.ptr(self.y), C._I(b), C._I(at.n_head), C._I(tmax),
                   C._F(at.scale), C._I(at.window // 128), L.stream())
            if self.split:
                x = self._lin(self.y, at.c_proj.weight, 1, x)
                x, xn = ops.norm_split(x)
                if self.dense[i]:
                    x = self._lin(self._lin(xn, blk.mlp.c_fc.weight, 2), blk.mlp.c_proj.weight, 1, x)
                else:
                    x = blk.mlp(xn.view(b, 1, -1), residual=x.view(b, 1, -1)).view(b, -1)
            else:
                x = ops.linear(self.y, at.c_proj.weight, residual=x)
                x, xn = ops.norm_split(x)
                x = blk.mlp(xn.view(b, 1, -1), residual=x.view(b, 1, -1)).view(b, -1) if not self.dense[i] else blk.mlp(xn, residual=x)
            if n_skip and i < n_skip:
                skips.append(x)
        xn = ops.rms_norm(x)
        logits = C.mm_nt(xn, model.lm_head.weight, epi=L.EPI_SOFTCAP, alpha=1.0 / cfg.softcap, beta=cfg.softcap)
        self.last_logits = logits                                          # [B, padded vocab] bf16, soft-capped
        nxt = logits[:, :cfg.vocab_size].float().argmax(-1)
        pos.add_(1)
        at = pos.to(torch.int64)
        forced = self.out.index_select(1, at)[:, 0]
        nxt = torch.where((pos < self.prompt_len).expand_as(nxt), forced, nxt)
        self.out.index_copy_(1, at, nxt[:, None])                         # token at position pos (after the increment)
        tok.copy_(nxt)

    @torch.no_grad()
    def run(self, n_steps: int):
        """``n_steps`` decode steps; the first one runs eagerly (it also warms every kernel up), the rest replay the graph."""
        if n_steps <= 0:
            return
        self._step()
        if n_steps == 1:
            return
        if self.graph is None:
            torch.cuda.synchronize()
            self.graph = torch.cuda.CUDAGraph()
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                with torch.cuda.graph(self.graph, stream=side):
                    self._step()
            torch.cuda.current_stream().wait_stream(side)       # capturing does not execute the step
        for _ in range(n_steps - 1):
            self.graph.replay()


@torch.no_grad()
def greedy_decode(model, prompts: torch.Tensor, n_new: int) -> torch.Tensor:
    """``prompts [B, P]`` -> ``[B, P + n_new]`` by arg-max decoding."""
    b, p = prompts.shape
    if p + n_new > model.config.sequence_len:
        raise ValueError("prompt + new tokens exceed the model's sequence length")
    if getattr(model, "os1", None) is not None or any(blk.attn is None for blk in model.transformer.h):
        return greedy_decode_full(model, prompts, n_new)          # output table and attention-free blocks: cache-free route
    cache = KVCache(model, b, p + n_new)
    if NativeDecoder.eligible(model) and n_new >= 1:
        out = torch.zeros(b, p + n_new, dtype=torch.int64, device=prompts.device)
        out[:, :p] = prompts
        if p <= 512:
            # short prompts are pre-filled token by token through the same graph (teacher-forced), then decoded
            dec = NativeDecoder(model, cache, prompts[:, 0], out, prompt_len=p)
            dec.run(p + n_new - 1)
        else:
            # long prompts: prefill on the cached PyTorch route, then one graph replay per generated token
            logits = _forward_cached(model, prompts, cache)
            first = logits.argmax(-1)
            out[:, p] = first
            if n_new > 1:
                dec = NativeDecoder(model, cache, first, out)
                dec.run(n_new - 1)
        L_check()
        return out
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
