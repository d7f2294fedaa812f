"""Evaluation helpers that stand in for the competition kit's ``evaluate_bpb`` and ``causality_check`` (absent from
the reference repository; used at round2/source/train.py:23307-23318).

* ``evaluate_bpb``     -- bits per byte = sum(nats) / (ln 2 * sum(bytes)) over a held-out synthetic stream with a fixed
  bytes-per-token table; BOS targets are excluded like in training.
* ``causality_check``  -- perturb tokens at positions > p and require the logits at positions <= p to stay put.  This
  also covers the MoE capacity count and the hashed-table lookups, which are causal by construction.
* ``score_continuations`` -- teacher-forced log-likelihood of a continuation given a context (the scoring half of the
  inference benchmark).
"""
from __future__ import annotations

import math
import time

import torch

from ..data.synth import SynthLoader, bytes_per_token_table


@torch.no_grad()
def evaluate_bpb(model, vocab: int, batch: int, seq_len: int, device, *, max_tokens: int = 1 << 20, seed: int = 1234,
                 timeout_seconds: float = 1e9, bos_id: int = 0) -> dict:
    loader = SynthLoader(vocab, seq_len, batch, rank=0, seed=seed, bos_id=bos_id)
    nbytes = bytes_per_token_table(vocab).to(device)
    t0 = time.time()
    nats, total_bytes, ntok = 0.0, 0, 0
    was_training = model.training
    model.eval()
    timed_out = False
    while ntok < max_tokens:
        x, y = loader.next_step()
        x, y = x.to(device), y.to(device)
        nll = model(x.long() if device.type == "cpu" else x, y, loss_reduction="none")
        valid = y >= 0
        nats += float((nll * valid).sum())
        total_bytes += int((nbytes[y.clamp_min(0)] * valid).sum())
        ntok += int(valid.sum())
        if time.time() - t0 > timeout_seconds:
            timed_out = True
            break
    model.train(was_training)
    return dict(val_bpb=nats / (math.log(2) * max(total_bytes, 1)), eval_seconds=time.time() - t0, num_tokens=ntok,
                eval_timeout=timeout_seconds, eval_over_timeout=timed_out)


@torch.no_grad()
def causality_check(model, vocab: int, batch: int, seq_len: int, device, seed: int = 7) -> dict:
    g = torch.Generator().manual_seed(seed)
    x = torch.randint(1, vocab, (batch, seq_len), generator=g)
    cut = seq_len // 2
    x2 = x.clone()
    x2[:, cut:] = torch.randint(1, vocab, (batch, seq_len - cut), generator=g)
    was_training = model.training
    model.eval()
    a = model(x.to(device)).float()
    b = model(x2.to(device)).float()
    model.train(was_training)
    diff = float((a[:, :cut] - b[:, :cut]).abs().max())
    tol = 1e-4 if a.device.type == "cpu" else 5e-2
    return dict(passed=diff <= tol, max_abs_diff=diff)


@torch.no_grad()
def score_continuations(model, tokens: torch.Tensor, ctx_len: torch.Tensor, total_len: torch.Tensor) -> torch.Tensor:
    """``tokens [B, T]`` padded; request b's context is ``tokens[b, :ctx_len[b]]`` and its continuation
    ``tokens[b, ctx_len[b]:total_len[b]]``.  Returns the summed log-probability of each continuation."""
    b, t = tokens.shape
    targets = torch.full((b, t), -1, dtype=torch.int64, device=tokens.device)
    targets[:, :-1] = tokens[:, 1:]
    pos = torch.arange(t, device=tokens.device)[None, :]
    keep = (pos + 1 >= ctx_len[:, None]) & (pos + 1 < total_len[:, None])
    targets = torch.where(keep, targets, torch.full_like(targets, -1))
    nll = model(tokens, targets, loss_reduction="none")
    return -(nll * keep).sum(1)
