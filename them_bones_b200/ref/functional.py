"""Plain-PyTorch statement of every operator in the framework.

These functions are (a) the CPU execution path, (b) the numerical oracle every CUDA kernel is tested against and
(c) the cuBLAS/SDPA/NCCL baseline path on a GPU.  They restate the reference's eager expressions (the expressions
its accelerated kernels replace and keep as fallbacks): ``norm`` round2/source/train.py:4570, ``apply_rotary_emb``
:4726-4731, attention :10209-10252, ReLU^2 MLP :10255-10300, softcap + cross-entropy :11688-11702, residual mix
:11070-11079, Muon/AdamW math :11783-11967, MoE routing :10505-10600.
"""
from __future__ import annotations

import math

import torch
import torch.nn.functional as F

# ----------------------------------------------------------------------------------------------------------------
# normalisation / residual / rotary
# ----------------------------------------------------------------------------------------------------------------

RMS_EPS = 2.0 ** -23


def rms_norm(x: torch.Tensor, eps: float = RMS_EPS) -> torch.Tensor:
    """Parameter-free RMSNorm over the last dim, computed in fp32."""
    xf = x.float()
    return (xf * torch.rsqrt(xf.square().mean(-1, keepdim=True) + eps)).to(x.dtype)


def shift1(x: torch.Tensor) -> torch.Tensor:
    """Causal one-token shift over the sequence dim of ``[B, T, C]``: row t is input row t-1, row 0 is zeros
    (reference: round1/source/train.py:300-304)."""
    return torch.cat((x.new_zeros(x.shape[0], 1, x.shape[2]), x[:, :-1, :]), dim=1)


def resid_mix(x, x0, a, b):
    """``x = a * x + b * x0`` with scalar gains."""
    return (a.float() * x.float() + b.float() * x0.float()).to(x.dtype)


def rotary_tables(seq_len: int, head_dim: int, base: float, dtype=torch.float32, device=None):
    """cos/sin ``[T, head_dim/2]`` rounded to ``dtype`` (the reference rounds its tables to the compute dtype)."""
    freqs = torch.arange(0, head_dim, 2, dtype=torch.float32, device=device)
    inv_freq = 1.0 / (base ** (freqs / head_dim))
    t = torch.arange(seq_len, dtype=torch.float32, device=device)
    table = torch.outer(t, inv_freq)
    return table.cos().to(dtype), table.sin().to(dtype)


def apply_rotary(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """Rotate-half RoPE on ``x [B, T, H, D]``: ``y1 = x1 cos + x2 sin; y2 = -x1 sin + x2 cos``."""
    d = x.shape[-1] // 2
    x1, x2 = x[..., :d].float(), x[..., d:].float()
    c, s = cos[None, :x.shape[1], None, :].float(), sin[None, :x.shape[1], None, :].float()
    return torch.cat([x1 * c + x2 * s, -x1 * s + x2 * c], dim=-1).to(x.dtype)


# ----------------------------------------------------------------------------------------------------------------
# attention
# ----------------------------------------------------------------------------------------------------------------

def doc_start_positions(idx: torch.Tensor, bos_id: int) -> torch.Tensor:
    """For every position of ``idx [B, T]`` the position of the most recent BOS at or before it (0 when the window
    starts mid-document).  A query may only attend keys at positions >= this value."""
    b, t = idx.shape
    pos = torch.arange(t, device=idx.device, dtype=torch.int32).expand(b, t)
    marks = torch.where(idx == bos_id, pos, torch.zeros_like(pos))
    return torch.cummax(marks, dim=1).values.to(torch.int32)


def attention_mask(t: int, device, doc_start: torch.Tensor | None = None, window: int = 0) -> torch.Tensor:
    """Boolean ``[B or 1, 1, T, T]`` mask (True = attend): causal, optionally limited to the query's document and to
    a band of 128-token tiles (keys in the query's tile and the ``window/128 - 1`` tiles before it; reference:
    ``attn_band_mask``, round2/source/train.py:4740-4745)."""
    q = torch.arange(t, device=device)[:, None]
    k = torch.arange(t, device=device)[None, :]
    m = (k <= q)
    if window:
        nw = window // 128
        m = m & ((q // 128 - k // 128) < nw)
    m = m[None, None]
    if doc_start is not None:
        m = m & (k[None, None] >= doc_start[:, None, :, None].to(torch.int64))
    return m


def attention(qkv: torch.Tensor, cos, sin, n_head: int, head_dim: int, scale: float,
              doc_start: torch.Tensor | None = None, window: int = 0) -> torch.Tensor:
    """Fused-op semantics: packed ``qkv [B, T, 3*H*D]`` -> RoPE(q, k) -> RMS-norm(q, k) -> masked softmax attention ->
    ``[B, T, H*D]``.  Math in fp32."""
    b, t, _ = qkv.shape
    c = n_head * head_dim
    q, k, v = qkv.split(c, dim=-1)
    q = rms_norm(apply_rotary(q.reshape(b, t, n_head, head_dim), cos, sin))
    k = rms_norm(apply_rotary(k.reshape(b, t, n_head, head_dim), cos, sin))
    v = v.reshape(b, t, n_head, head_dim)
    qf, kf, vf = (z.transpose(1, 2).float() for z in (q, k, v))
    s = torch.matmul(qf, kf.transpose(-1, -2)) * scale
    mask = attention_mask(t, qkv.device, doc_start, window)
    s = s.masked_fill(~mask, float("-inf"))
    p = torch.softmax(s, dim=-1)
    y = torch.matmul(p, vf).transpose(1, 2).reshape(b, t, c)
    return y.to(qkv.dtype)


# ----------------------------------------------------------------------------------------------------------------
# MLP, loss
# ----------------------------------------------------------------------------------------------------------------

def relu2(x):
    return F.relu(x).square()


def mlp(x, w_fc, w_proj):
    return F.linear(relu2(F.linear(x, w_fc)), w_proj)


def softcap_logits(logits: torch.Tensor, cap: float) -> torch.Tensor:
    return cap * torch.tanh(logits.float() / cap)


def softcap_cross_entropy(x: torch.Tensor, w: torch.Tensor, targets: torch.Tensor, vocab: int, cap: float,
                          weights: torch.Tensor | None = None, reduction: str = "mean", label_smoothing: float = 0.0):
    """lm_head GEMM + fp32 softcap + cross-entropy with ``ignore_index=-1``.  ``weights`` (per row) gives the
    row-weighted sum form of the chunked loss head (reference: ``chunked_loss_mean``, round2/source/train.py:6364)."""
    logits = softcap_logits(F.linear(x, w)[..., :vocab], cap)
    flat, tgt = logits.reshape(-1, vocab), targets.reshape(-1)
    if weights is not None:
        nll = F.cross_entropy(flat, tgt, ignore_index=-1, reduction="none", label_smoothing=label_smoothing)
        return (nll * weights.reshape(-1).float()).sum()
    out = F.cross_entropy(flat, tgt, ignore_index=-1, reduction=reduction, label_smoothing=label_smoothing)
    return out.view_as(targets) if reduction == "none" else out


# ----------------------------------------------------------------------------------------------------------------
# MXFP8 (OCP microscaling): 1x32 blocks along the contraction axis, UE8M0 scales, E4M3 elements
# ----------------------------------------------------------------------------------------------------------------

E4M3_MAX = 448.0
MX_BLOCK = 32


def mx_scale_exponent(amax: torch.Tensor) -> torch.Tensor:
    """Biased UE8M0 exponent for a block with absolute maximum ``amax``: the smallest power of two ``2**e`` with
    ``amax / 2**e <= 448`` (round the scale up so nothing saturates); an all-zero block gets exponent 0 -> 2**-127."""
    a = amax.float().clamp_min(0)
    e = torch.ceil(torch.log2(a / E4M3_MAX))
    e = torch.where(a > 0, e, torch.full_like(e, -127.0))
    # guard against log2 rounding: step up while a / 2**e > 448
    e = torch.where(a > E4M3_MAX * torch.exp2(e), e + 1, e)
    return (e.clamp(-127, 127) + 127).to(torch.uint8)


def mx_quantize(x: torch.Tensor, axis: int = -1):
    """Quantise along ``axis`` in blocks of 32.  Returns ``(q float8_e4m3fn same shape, scales uint8 [..., n/32])``
    with the block axis moved last in ``scales``."""
    xm = x.float().movedim(axis, -1)
    shp = xm.shape
    blk = xm.reshape(*shp[:-1], shp[-1] // MX_BLOCK, MX_BLOCK)
    e = mx_scale_exponent(blk.abs().amax(-1))
    scale = torch.exp2(e.float() - 127.0).unsqueeze(-1)
    q = (blk / scale).clamp(-E4M3_MAX, E4M3_MAX).to(torch.float8_e4m3fn)
    return q.reshape(shp).movedim(-1, axis), e


def mx_dequantize(q: torch.Tensor, e: torch.Tensor, axis: int = -1) -> torch.Tensor:
    qm = q.float().movedim(axis, -1)
    shp = qm.shape
    blk = qm.reshape(*shp[:-1], shp[-1] // MX_BLOCK, MX_BLOCK)
    out = blk * torch.exp2(e.float() - 127.0).unsqueeze(-1)
    return out.reshape(shp).movedim(-1, axis)


def mx_qdq(x: torch.Tensor, axis: int = -1) -> torch.Tensor:
    """Quantise-dequantise: the value an MXFP8 GEMM sees for ``x``."""
    q, e = mx_quantize(x, axis)
    return mx_dequantize(q, e, axis)


def mx_linear(x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """Rounding-exact emulation of the block-scaled GEMM ``x @ w.T``: both operands quantised along K, products
    accumulated in fp32, result rounded to ``x.dtype``."""
    return (mx_qdq(x, -1) @ mx_qdq(w, -1).T).to(x.dtype)


def mx_mlp(x, w_fc, w_proj):
    """MXFP8 MLP forward: c_fc GEMM -> ReLU^2 in fp32 on the accumulator -> re-quantised along the hidden axis ->
    c_proj GEMM."""
    pre = mx_qdq(x, -1) @ mx_qdq(w_fc, -1).T
    h = F.relu(pre).square()
    return (mx_qdq(h, -1) @ mx_qdq(w_proj, -1).T).to(x.dtype)


# ----------------------------------------------------------------------------------------------------------------
# Muon pieces
# ----------------------------------------------------------------------------------------------------------------

POLAR_EXPRESS_COEFFS = [
    (8.156554524902461, -22.48329292557795, 15.878769915207462),
    (4.042929935166739, -2.808917465908714, 0.5000178451051316),
    (3.8916678022926607, -2.772484153217685, 0.5060648178503393),
    (3.285753657755655, -2.3681294933425376, 0.46449024233003106),
    (2.3465413258596377, -1.7097828382687081, 0.42323551169305323),
]


def newton_schulz(x: torch.Tensor, steps: int = 5) -> torch.Tensor:
    """Polar-Express Newton-Schulz on a stack ``[n, r, c]`` already normalised by its Frobenius norm.  Tall matrices
    iterate on ``X^T X`` (c x c), wide ones on ``X X^T``."""
    if x.shape[-2] > x.shape[-1]:
        for a, b, c in POLAR_EXPRESS_COEFFS[:steps]:
            g = x.mT @ x
            x = a * x + x @ (b * g + c * (g @ g))
    else:
        for a, b, c in POLAR_EXPRESS_COEFFS[:steps]:
            g = x @ x.mT
            x = a * x + (b * g + c * (g @ g)) @ x
    return x


def muon_update(g, w, momentum_buffer, second, *, momentum, beta2, lr, wd, ns_steps=5, ns_dtype=torch.float32,
                ns_fn=None):
    """One Muon step on stacks ``[n, r, c]`` (in place on ``w``, ``momentum_buffer``, ``second``): momentum lerp,
    Nesterov, Frobenius normalisation, Polar-Express NS, NorMuon second-moment rescale that keeps the Frobenius norm,
    cautious weight decay, ``lr * sqrt(max(1, r/c))`` (reference: round2/source/train.py:11868-11905)."""
    r, c = g.shape[-2:]
    lr_eff = lr * max(1.0, r / c) ** 0.5
    momentum_buffer.lerp_(g, 1 - momentum)
    g = g.lerp(momentum_buffer, momentum)
    x = g.to(ns_dtype)
    x = x / (x.norm(dim=(-2, -1), keepdim=True) * 1.01 + 1e-6)
    g = (ns_fn or newton_schulz)(x.contiguous() if ns_fn else x, ns_steps)
    red_dim = -1 if r >= c else -2
    v_mean = g.float().square().mean(dim=red_dim, keepdim=True)
    n_red = g.size(red_dim)
    v_norm = (v_mean.sum(dim=(-2, -1), keepdim=True) * n_red).sqrt()
    second.lerp_(v_mean, 1 - beta2)
    step_size = second.clamp_min(1e-10).rsqrt()
    scaled = (v_mean * n_red) * step_size.square()
    v_norm_new = scaled.sum(dim=(-2, -1), keepdim=True).sqrt()
    g = g.float() * (step_size * (v_norm / v_norm_new.clamp_min(1e-10)))
    mask = (g * w.float()) >= 0
    w.sub_((lr_eff * g + lr_eff * wd * w.float() * mask).to(w.dtype))
    return w


def adamw_update(p, grad, exp_avg, exp_avg_sq, *, step, lr, beta1, beta2, eps, wd):
    """Decoupled-decay AdamW with bias correction (reference: round2/source/train.py:11803-11832)."""
    p.mul_(1 - lr * wd)
    exp_avg.lerp_(grad, 1 - beta1)
    exp_avg_sq.lerp_(grad.square(), 1 - beta2)
    b1, b2 = 1 - beta1 ** step, 1 - beta2 ** step
    p.sub_(lr * (exp_avg / b1) / ((exp_avg_sq / b2).sqrt() + eps))
    return p


# ----------------------------------------------------------------------------------------------------------------
# MoE routing (capacity-limited, causal within a sequence)
# ----------------------------------------------------------------------------------------------------------------

def moe_route(logits: torch.Tensor, topk: int):
    """fp32 router logits ``[N, E]`` -> ``(p [N,E], idx [N,k] int64, gates [N,k])``.  Top-1 gate is the probability
    itself; top-2 gates are renormalised over the two.  Ties go to the lower expert index."""
    p = torch.softmax(logits.float(), dim=-1)
    n, e = p.shape
    i1 = torch.argmax(p, dim=-1)                               # first maximum
    v1 = p.gather(1, i1[:, None])[:, 0]
    if topk == 1:
        return p, i1[:, None], v1[:, None]
    p2 = p.detach().scatter(1, i1[:, None], -1.0)
    i2 = torch.argmax(p2, dim=-1)
    v2 = p.gather(1, i2[:, None])[:, 0]
    den = v1 + v2
    return p, torch.stack([i1, i2], 1), torch.stack([v1 / den, v2 / den], 1)


def moe_slots(idx: torch.Tensor, b: int, t: int, n_exp: int, cap: int):
    """Causal per-sequence capacity.  ``idx [b*t, k]`` -> ``slot [b*t, k]`` int64 in the ``[E, b, cap]`` buffer (or
    ``E*b*cap`` when the assignment is dropped) and ``token_of_slot [E*b*cap]`` (or ``b*t`` when empty).  Position of
    an assignment = number of assignments to the same expert at earlier positions of the same sequence (a token's k
    choices are distinct experts; reference: ``moe_positions``/``moe_gather_tables``,
    round2/source/train.py:10555-10636)."""
    n, k = idx.shape
    total = n_exp * b * cap
    onehot = torch.zeros(n, n_exp, dtype=torch.int64, device=idx.device)
    onehot.scatter_add_(1, idx, torch.ones_like(idx))
    incl = onehot.view(b, t, n_exp).cumsum(1)
    excl = (incl - onehot.view(b, t, n_exp)).view(n, n_exp)
    pos = excl.gather(1, idx)                                  # [n, k]
    row = (torch.arange(n, device=idx.device) // t)[:, None]
    keep = pos < cap
    slot = torch.where(keep, (idx * b + row) * cap + pos, torch.full_like(pos, total))
    tok = torch.full((total + 1,), n, dtype=torch.int64, device=idx.device)
    src = torch.arange(n, device=idx.device)[:, None].expand(n, k)
    tok.scatter_(0, slot.reshape(-1), src.reshape(-1))
    tok = tok[:total]
    return slot, tok


def moe_aux_terms(p, logits, idx, n_exp: int, topk: int, aux_w: float, z_w: float):
    """Switch load-balance term ``E * sum_e f_e P_e`` (f from the assignments, no gradient) and router z-loss
    (reference: ``moe_aux_terms``, round2/source/train.py:10779-10793)."""
    onehot = F.one_hot(idx, n_exp).sum(1).float()
    f = onehot.mean(0) / topk
    lb = n_exp * (f * p.mean(0)).sum()
    z = torch.logsumexp(logits.float(), dim=-1).square().mean()
    return aux_w * lb + z_w * z, lb, z, f


# ----------------------------------------------------------------------------------------------------------------
# hashed n-gram tables
# ----------------------------------------------------------------------------------------------------------------

HASH_MULT = (0x9E3779B97F4A7C15, 0xC2B2AE3D27D4EB4F, 0x165667B19E3779F9)
_MASK64 = (1 << 64) - 1


def _as_i64(v: int) -> int:
    v &= _MASK64
    return v - (1 << 64) if v >= (1 << 63) else v


def _ngram_hash(toks, order: int, rows: int, seed: int) -> torch.Tensor:
    """``toks[j]``: the token ``j`` places back (``j = 0`` the current one), already replaced by the pad id where the
    context does not reach that far.  All int64, same shape."""
    h = torch.full_like(toks[0], _as_i64(seed * 0x9E3779B97F4A7C15 + order))
    for j in range(order):
        h = (h ^ (toks[j] + 1)) * _as_i64(HASH_MULT[j % 3])
        h = h ^ ((h >> 29) & ((1 << 35) - 1))                 # logical shift of the wrapped value
    h = h * _as_i64(HASH_MULT[2])
    return ((h >> 32) & (rows - 1)).to(torch.int64) if rows <= (1 << 32) else (h & (rows - 1))


def ngram_rows(idx: torch.Tensor, order: int, rows: int, seed: int, doc_start: torch.Tensor | None = None,
               pad_id: int = 0) -> torch.Tensor:
    """Row index for every position of ``idx [B, T]``: a 64-bit multiplicative hash of the previous ``order`` token
    ids (the current token and ``order-1`` before it), reduced mod ``rows`` (a power of two).  Positions before the
    window start (or before the document start when ``doc_start`` is given) use ``pad_id``; the lookup is therefore
    causal.  Integer arithmetic wraps mod 2**64 identically on every platform."""
    b, t = idx.shape
    x = idx.to(torch.int64)
    pos = torch.arange(t, device=idx.device)[None, :]
    toks = []
    for j in range(order):
        tok = F.pad(x, (j, 0), value=pad_id)[:, :t]
        if doc_start is not None:
            tok = torch.where(pos - j >= doc_start.to(torch.int64), tok, torch.full_like(tok, pad_id))
        else:
            tok = torch.where(pos - j >= 0, tok, torch.full_like(tok, pad_id))
        toks.append(tok)
    return _ngram_hash(toks, order, rows, seed)


def ngram_rows_at(history: torch.Tensor, pos: torch.Tensor, order: int, rows: int, seed: int,
                  doc_start: torch.Tensor | None = None, pad_id: int = 0) -> torch.Tensor:
    """The same row index for the single position ``pos`` (a device scalar) of ``history [B, L]`` (the tokens so far):
    what a decode step needs, with no host read of the position.  ``doc_start [B]``: first position of each sequence's
    current document."""
    b = history.shape[0]
    toks = []
    for j in range(order):
        at = (pos.to(torch.int64) - j).reshape(1)
        tok = history.index_select(1, at.clamp_min(0))[:, 0].to(torch.int64)
        lo = doc_start.to(torch.int64) if doc_start is not None else torch.zeros(b, dtype=torch.int64, device=history.device)
        toks.append(torch.where(at.expand(b) >= lo, tok, torch.full_like(tok, pad_id)))
    return _ngram_hash(toks, order, rows, seed)


# ----------------------------------------------------------------------------------------------------------------
# Output-side hashed table ("OS1"): keys, signs, codebook, gate, readout, row update
# (reference: switch 59, round2/source/train.py:2310-2351 and the helpers at :2596-2680)
# ----------------------------------------------------------------------------------------------------------------

def _lsr(z: torch.Tensor, s: int) -> torch.Tensor:
    """Logical right shift of int64 values holding wrapped 64-bit words."""
    return (z >> s) & ((1 << (64 - s)) - 1)


def _mix64(z: torch.Tensor) -> torch.Tensor:
    """A splitmix64-style finaliser on wrapped int64 words."""
    z = (z ^ _lsr(z, 30)) * _as_i64(0xBF58476D1CE4E5B9)
    z = (z ^ _lsr(z, 27)) * _as_i64(0x94D049BB133111EB)
    return z ^ _lsr(z, 31)


def os1_keys(idx: torch.Tensor, order: int, rows: int, bos_id: int, seed: int = 0):
    """For token ids ``[B, T]``: ``(row [B, T] int64, -1 where no key exists; sign_hash [B, T] int64)`` of the ``order``
    ids ending at each position.  A key exists where all ``order`` ids lie in the window and none after the first is
    BOS (reference: ``os1_keys``, round2/source/train.py:2596-2624, there with tabulation hashing on the host; here two
    position-salted multiplicative hashes computed on the tokens' device)."""
    b, t = idx.shape
    x = idx.to(torch.int64)
    h0 = torch.full((b, t), _as_i64(seed * HASH_MULT[0] + 0x51ED270B), dtype=torch.int64, device=idx.device)
    h1 = torch.full((b, t), _as_i64(seed * HASH_MULT[1] + 0x2545F491), dtype=torch.int64, device=idx.device)
    for j in range(min(order, t)):
        tok = F.pad(x, (j, 0), value=0)[:, :t] + 1
        h0 = _mix64(h0 + tok * _as_i64(HASH_MULT[j % 3]) + j)
        h1 = _mix64(h1 ^ (tok * _as_i64(HASH_MULT[(j + 1) % 3]) + 7 * j))
    c = (x == bos_id).to(torch.int64).cumsum(1)
    prev = torch.zeros_like(c)
    if order - 1 < t:
        prev[:, order - 1:] = c[:, :t - order + 1]
    pos = torch.arange(t, device=idx.device)[None, :]
    valid = (pos >= order - 1) & (c - prev == 0)
    row = torch.where(valid, _lsr(h0, 8) & (rows - 1), torch.full_like(h0, -1))
    return row, h1


def os1_signs(hsign: torch.Tensor, dim: int) -> torch.Tensor:
    """``dim`` signs (+1 / -1, fp32 ``[n, dim]``) of each sign hash ``[n]``: the bits, low first, of mixed words
    ``mix(hash + (k + 1) * golden)``, one word per 64 signs (reference: ``os1_signs``, round2/source/train.py:2627-2643)."""
    h = hsign.reshape(-1, 1)
    words = (dim + 63) // 64
    gold = torch.tensor([_as_i64((k + 1) * 0x9E3779B97F4A7C15) for k in range(words)], dtype=torch.int64, device=h.device)
    z = _mix64(h + gold[None, :])                                             # [n, words]
    sh = torch.arange(64, dtype=torch.int64, device=h.device)
    bits = (z[:, :, None] >> sh[None, None, :]) & 1                           # arithmetic shift, low bit kept
    return (1 - 2 * bits).reshape(h.shape[0], words * 64)[:, :dim].to(torch.float32)


def os1_codebook(vocab_pad: int, dim: int, seed: int) -> torch.Tensor:
    """Fixed readout codebook, fp32 ``[vocab_pad, dim]`` unit rows from a generator of its own (reference:
    ``os1_codebook``, round2/source/train.py:2646-2651)."""
    g = torch.Generator().manual_seed(seed)
    c = torch.randn(vocab_pad, dim, generator=g, dtype=torch.float32)
    return c / c.norm(dim=1, keepdim=True)


def os1_gate(u: torch.Tensor, code: torch.Tensor, idx: torch.Tensor, a0: float, width: int, h0: float, slope: float):
    """Gate ``G [B, T]`` = sigmoid(slope * (h - h0)), ``h_t`` the mean over the previous ``width`` positions j of the
    window of ``s_j`` read at the token that followed j (an input at t, so the gate is causal); ``h_0 = 0``.  No
    gradient flows through it (reference: the banded mean ``os1_band``, round2/source/train.py:2654-2661)."""
    with torch.no_grad():
        b, t = idx.shape
        nxt = idx[:, 1:].reshape(-1)
        uu = u.view(b, t, -1)[:, :-1].reshape(-1, u.shape[-1]).float()
        sd = (uu * code.index_select(0, nxt).float()).sum(-1).view(b, t - 1) / a0       # s_j at token j+1, j < T-1
        cs = F.pad(sd.cumsum(1), (1, 0))                                               # cs[t] = sum_{j<t} sd[j]
        pos = torch.arange(t, device=idx.device)
        lo = (pos - width).clamp_min(0)
        n = (pos - lo).clamp_min(1).float()
        h = (cs[:, pos] - cs[:, lo]) / n
        return torch.sigmoid(slope * (h - h0))


def os1_readout(s: torch.Tensor, gate: torch.Tensor, glin: float, beta: float, thr: float) -> torch.Tensor:
    """Additive pre-softcap logit term for scores ``s [M, V]`` and gate ``[M]``:
    ``glin * s + G * beta * relu(sg(s) - thr) / (1 - thr)`` (reference: round2/source/train.py:2321-2323)."""
    return glin * s + gate[:, None] * (beta / (1.0 - thr)) * torch.relu(s.detach() - thr)


def os1_row_step(x: torch.Tensor, g: torch.Tensor, lr: float, eps: float, cap: float) -> torch.Tensor:
    """The table's stateless update on rows ``x [n, dim]`` with summed gradients ``g``: ``x - lr g / (rms(g) + eps)``,
    then scaled back onto ``rms(x) <= cap * lr`` (reference: ``os1_row_step``, round2/source/train.py:2671-2680).
    Returns the new rows (fp32)."""
    x, g = x.float(), g.float()
    r = g.square().mean(1, keepdim=True).sqrt()
    x = x - g * (lr / (r + eps))
    q = x.square().mean(1, keepdim=True).sqrt()
    return x * torch.clamp((cap * lr) / q.clamp_min(1e-30), max=1.0)


def os1_typ_rms(glin: float, a0: float, dim: int, tokens: int, world: int) -> float:
    """RMS of one position's row gradient when ``|C^T d(logits)| = 1`` under the mean loss over ``tokens`` and the
    average over ``world`` ranks (reference: ``os1_typ_rms``, round2/source/train.py:2664-2668)."""
    return glin / (a0 * math.sqrt(dim) * max(1, tokens) * max(1, world))


def softcap_cross_entropy_os1(x, w, targets, vocab, cap, u, code, gate, *, a0, glin, beta, thr, weights=None,
                              reduction="mean"):
    """``softcap_cross_entropy`` with the output table's term added before the soft-cap."""
    s = F.linear(u.to(x.dtype), code.to(x.dtype)).float()[..., :vocab] / a0
    pre = F.linear(x, w).float()[..., :vocab].reshape(-1, vocab) + os1_readout(s.reshape(-1, vocab), gate.reshape(-1), glin, beta, thr)
    flat, tgt = softcap_logits(pre, cap), targets.reshape(-1)
    if weights is not None:
        nll = F.cross_entropy(flat, tgt, ignore_index=-1, reduction="none")
        return (nll * weights.reshape(-1).float()).sum()
    out = F.cross_entropy(flat, tgt, ignore_index=-1, reduction=reduction)
    return out.view_as(targets) if reduction == "none" else out


# ----------------------------------------------------------------------------------------------------------------
# Packed views of table rows: the forward reads a 1-bit or 4-bit view of the master row, the gradient goes straight
# through to the master, and the checkpoint stores the view itself
# (reference: R2_NGRAM_BITS, round2/source/train.py:1016-1029; R2_OS1_BITS, :2371-2390 and helpers :2692-2732)
# ----------------------------------------------------------------------------------------------------------------

def _bf16_round_up(x: torch.Tensor) -> torch.Tensor:
    """Positive fp64 values to the nearest bf16 value that is not below them (up to a 1e-12 relative slack, so that a
    value that is a bf16 number up to the last bits of its fp64 computation maps to itself on every device)."""
    b = x.to(torch.bfloat16)
    low = b.double() < x * (1.0 - 1e-12)
    bumped = (b.view(torch.int16) + 1).view(torch.bfloat16)
    return torch.where(low, bumped, b)


def table_view_scale(rows: torch.Tensor, bits: int) -> torch.Tensor:
    """Per-row scale ``[n, 1]`` (bf16-representable fp32) of the ``bits``-bit view: the mean ``|value|`` (1 bit) or
    ``max |value| / 7`` rounded up to bf16 (4 bits)."""
    m = rows.float()
    if bits == 1:
        return m.abs().mean(1, keepdim=True).to(torch.bfloat16).float()
    if bits == 4:
        # in fp64: a back end may turn the division by a constant into a multiplication, and the scale must come out
        # the same on every device and map a view onto itself
        return _bf16_round_up(m.abs().amax(1, keepdim=True).double() / 7.0).float()
    raise ValueError(f"view bits {bits}: 1 or 4")


def table_view(rows: torch.Tensor, bits: int) -> torch.Tensor:
    """The view the forward reads, in the rows' dtype: ``sign(m) * s`` with ``sign(0) = +1`` (1 bit) or
    ``round(m / s) * s`` with levels -7..7 (4 bits); a zero row reads zero either way."""
    if bits == 0:
        return rows
    m, s = rows.float(), table_view_scale(rows, bits)
    if bits == 1:
        v = torch.where(m < 0, -s, s)
    else:
        v = torch.round(m / s.clamp_min(1e-30)).clamp(-7, 7) * s
    return v.to(rows.dtype)


def table_pack_view(rows: torch.Tensor, bits: int):
    """``(packed uint8 [n, dim * bits / 8], scale bf16 [n])`` of the view.  1 bit: sign bits eight to a byte along the
    width, bit k of byte j = column 8 j + k, 1 = negative.  4 bits: two levels to a byte, column 2 j in the low nibble,
    4-bit two's complement."""
    m, s = rows.float(), table_view_scale(rows, bits)
    n, dim = m.shape
    if bits == 1:
        neg = (m < 0).to(torch.uint8).view(n, dim // 8, 8)
        w = (1 << torch.arange(8, device=m.device)).to(torch.uint8)
        packed = (neg * w).sum(-1).to(torch.uint8)
    else:
        q = torch.round(m / s.clamp_min(1e-30)).clamp(-7, 7).to(torch.int16) & 0xF
        q = q.view(n, dim // 2, 2)
        packed = (q[..., 0] | (q[..., 1] << 4)).to(torch.uint8)
    return packed, s.reshape(n).to(torch.bfloat16)


def table_unpack_view(packed: torch.Tensor, scale: torch.Tensor, bits: int) -> torch.Tensor:
    """Inverse of ``table_pack_view``: the view's rows, fp32 ``[n, dim]``."""
    n = packed.shape[0]
    s = scale.float().reshape(n, 1)
    p = packed.to(torch.int16)
    if bits == 1:
        sh = torch.arange(8, device=packed.device)
        neg = ((p[..., None] >> sh) & 1).reshape(n, -1).bool()
        return torch.where(neg, -s, s)
    lo, hi = p & 0xF, (p >> 4) & 0xF
    q = torch.stack([lo, hi], -1).reshape(n, -1)
    q = torch.where(q >= 8, q - 16, q).float()
    return q * s


@torch.no_grad()
def table_rowrms_update(table, rows, g, row_sq, *, lr, beta, eps, decay, generator=None):
    """Row-wise RMS update of the touched rows (in place on ``table[rows]`` and ``row_sq[rows]``): one fp32 second moment
    per row, ``acc = beta acc + (1 - beta) mean(g^2)``, ``row = row (1 - decay) - lr g / (sqrt(acc) + eps)``; a bf16 table
    is written back with stochastic rounding (reference: ``NgramHostTable.step``, round2/source/train.py:3686-3701)."""
    a = row_sq.index_select(0, rows) * beta + (1.0 - beta) * g.float().square().mean(dim=1)
    row_sq.index_copy_(0, rows, a)
    w = table.index_select(0, rows).float() * (1.0 - lr * decay) - (lr / (a.sqrt() + eps)).unsqueeze(1) * g.float()
    table.index_copy_(0, rows, stochastic_round_bf16(w, generator) if table.dtype == torch.bfloat16 else w.to(table.dtype))


def stochastic_round_bf16(x: torch.Tensor, generator=None) -> torch.Tensor:
    """fp32 -> bf16 with stochastic rounding: a uniform 16-bit integer is added to the low half of the fp32 pattern
    before truncation, so the expected value of the result is ``x`` (the reference's bf16 master weights rely on the
    accelerator runtime's stochastic rounding, round1/source/train.py:10219-10226)."""
    bits = x.contiguous().view(torch.int32)
    r = torch.randint(0, 1 << 16, bits.shape, dtype=torch.int32, device=x.device, generator=generator)
    out = ((bits + r) & -65536).view(torch.float32)
    return torch.where(torch.isfinite(x), out, x).to(torch.bfloat16)
