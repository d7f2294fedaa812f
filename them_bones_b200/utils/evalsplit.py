"""Split evaluation: the held-out loss broken down by model-free position classes.

The reference attaches an observation-only hook to its scored forward (``EvalSplit``, round2/source/train.py:20777-21024)
that adds each target's nats, bytes and token count into classes read from a label file built from the eval stream
alone: *novel* text (no 8-token context match in the training text), near-duplicates, in-document bigram repeats.  The
classes answer "where does a table / a memorising component help".  Here the labels are computed from the streams
themselves (no file): every rank classifies the targets of its own eval windows with hashed context sets, accumulates
``[nats, bytes, tokens]`` per class on the host in float64 / int64, and rank 0 merges the ranks' sums
(one all-reduce) and prints one ``eval_split`` line.  The model is never changed and sees the same calls as
``evaluate_bpb``.

Classes of a target at position p (0-based in its window, target = token p + 1):
  ``bi_rep``   the bigram (token p, target) occurred earlier in the same document inside the window
  ``ctx_seen`` the ``ctx``-token context ending at p occurred in the reference stream given to ``ContextSet`` (training
               text), so a context-keyed table can have a row for it
  ``novel``    neither of the above
  ``all``      every valid target
"""
from __future__ import annotations

import json
import math

import numpy as np
import torch

_MULT = np.uint64(0x9E3779B97F4A7C15)


def _rolling_hash(tokens: np.ndarray, width: int) -> np.ndarray:
    """Hash of the ``width`` ids ending at each position of a 1-D stream (positions < width - 1 get 0 = "no context")."""
    t = tokens.astype(np.uint64) + np.uint64(1)
    n = len(t)
    h = np.zeros(n, dtype=np.uint64)
    with np.errstate(over="ignore"):
        for j in range(min(width, n)):
            part = np.zeros(n, dtype=np.uint64)
            part[j:] = t[:n - j]
            h = (h ^ part) * _MULT
            h ^= h >> np.uint64(29)
    h |= np.uint64(1)                       # a real context never hashes to the "no context" value
    h[:width - 1] = 0
    return h


class ContextSet:
    """The set of ``ctx``-token contexts of a reference stream (hashed; membership has no false negatives)."""

    def __init__(self, ctx: int = 8):
        self.ctx = ctx
        self.keys = np.zeros(0, dtype=np.uint64)

    def add(self, tokens: np.ndarray):
        h = _rolling_hash(np.asarray(tokens).reshape(-1), self.ctx)
        self.keys = np.union1d(self.keys, h[h != 0])

    def seen(self, windows: np.ndarray) -> np.ndarray:
        """``[n, T]`` bool: the context ending at each position of each window is in the set."""
        out = np.zeros(windows.shape, dtype=bool)
        for i, w in enumerate(windows):
            h = _rolling_hash(w, self.ctx)
            out[i] = (h != 0) & np.isin(h, self.keys)
        return out


def bigram_repeats(x: np.ndarray, y: np.ndarray, bos_id: int) -> np.ndarray:
    """``[n, T]`` bool: (x[p], y[p]) occurred at an earlier position of the same document in the window."""
    n, t = x.shape
    out = np.zeros((n, t), dtype=bool)
    for i in range(n):
        doc = np.cumsum(x[i] == bos_id)
        key = (doc.astype(np.int64) << 42) | (x[i].astype(np.int64) << 21) | np.maximum(y[i], 0).astype(np.int64)
        _, first = np.unique(key, return_index=True)
        rep = np.ones(t, dtype=bool)
        rep[first] = False
        out[i] = rep & (y[i] >= 0)
    return out


class SplitEval:
    NAMES = ("all", "bi_rep", "ctx_seen", "novel")

    def __init__(self, vocab: int, bos_id: int = 0, contexts: ContextSet | None = None, token_bytes: torch.Tensor | None = None):
        from ..data.synth import bytes_per_token_table
        self.bos_id, self.contexts = bos_id, contexts
        self.token_bytes = (token_bytes if token_bytes is not None else bytes_per_token_table(vocab)).cpu().numpy().astype(np.int64)
        self.acc = {k: [0.0, 0, 0] for k in self.NAMES}              # nats (float64), bytes, tokens
        self.calls = 0

    def observe(self, x: torch.Tensor, y: torch.Tensor, nll: torch.Tensor):
        """One scored call: inputs, targets (-1 = ignored) and the per-position loss ``[n, T]``."""
        xn, yn = x.cpu().numpy().astype(np.int64), y.cpu().numpy().astype(np.int64)
        nats = nll.detach().double().cpu().numpy()
        valid = yn >= 0
        nb = self.token_bytes[np.maximum(yn, 0)] * valid
        rep = bigram_repeats(xn, yn, self.bos_id)
        seen = self.contexts.seen(xn) & valid if self.contexts is not None else np.zeros_like(valid)
        masks = dict(all=valid, bi_rep=rep, ctx_seen=seen, novel=valid & ~rep & ~seen)
        for k, m in masks.items():
            a = self.acc[k]
            a[0] += float(nats[m].sum())
            a[1] += int(nb[m].sum())
            a[2] += int(m.sum())
        self.calls += 1

    def merged(self, group=None) -> dict:
        """Per-class totals over all ranks plus bits per byte and nats per token."""
        import torch.distributed as dist
        t = torch.tensor([[a[0], float(a[1]), float(a[2])] for a in (self.acc[k] for k in self.NAMES)], dtype=torch.float64)
        if dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1:
            dev = torch.device("cuda", torch.cuda.current_device()) if dist.get_backend(group) == "nccl" else torch.device("cpu")
            t = t.to(dev)
            dist.all_reduce(t, group=group)
            t = t.cpu()
        out = {}
        for k, (nats, nb, ntok) in zip(self.NAMES, t.tolist()):
            out[k] = dict(nats=nats, bytes=int(nb), tokens=int(ntok), bpb=nats / (math.log(2) * max(nb, 1.0)),
                          nats_per_token=nats / max(ntok, 1.0))
        return out

    def line(self, group=None) -> str:
        return "eval_split " + json.dumps(self.merged(group), separators=(",", ":"))


@torch.no_grad()
def evaluate_split(model, vocab: int, batch: int, seq_len: int, device, *, max_tokens: int = 1 << 18, seed: int = 1234,
                   bos_id: int = 0, contexts: ContextSet | None = None, rank: int = 0, group=None) -> dict:
    """The split evaluation over this rank's held-out synthetic stream (the stream ``evaluate_bpb`` scores when
    ``rank == 0``)."""
    from ..data.synth import SynthLoader
    loader = SynthLoader(vocab, seq_len, batch, rank=rank, seed=seed, bos_id=bos_id)
    ev = SplitEval(vocab, bos_id, contexts)
    was_training = model.training
    model.eval()
    ntok = 0
    while ntok < max_tokens:
        x, y = loader.next_step()
        xd, yd = x.to(device), y.to(device)
        nll = model(xd.long() if device.type == "cpu" else xd, yd, loss_reduction="none")
        ev.observe(x, y, nll)
        ntok += int((y >= 0).sum())
    model.train(was_training)
    return ev.merged(group)
