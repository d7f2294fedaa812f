"""Synthetic data pipeline: Zipf tokens in documents, best-fit packing, window slicing, BOS-target masking.

Stands in for the competition kit's ``make_dataloader`` (absent from the reference repository; its algorithm is
visible in the reference's own copy, round2/source/train.py:18945-19035): every document is ``BOS + tokens``; a row
of ``row_len + 1`` tokens is filled best-fit from a buffer of documents and, when nothing fits, the shortest
document is cropped into the remaining room; ``inputs = row[:-1]``, ``targets = row[1:]``.  One row per rank-step is
then cut into windows of ``seq_len`` tokens that may start mid-document (reference: window slicing,
round2/source/train.py:22006-22022) and targets equal to BOS are replaced by -1 (round2/source/train.py:22255-22256).

Token ids follow Zipf(s) over the vocabulary (rank r has probability proportional to r**-s) with id 0 reserved for
BOS, so ids are ``1 + rank``.  Everything is derived from one integer seed and the rank.
"""
from __future__ import annotations

import threading

import numpy as np
import torch


class ZipfDocs:
    """Endless stream of synthetic documents."""

    def __init__(self, vocab: int, s: float = 1.1, doc_len=(128, 2048), seed: int = 0, bos_id: int = 0):
        self.vocab, self.bos_id = vocab, bos_id
        self.lo, self.hi = doc_len
        self.rng = np.random.default_rng(seed)
        ranks = np.arange(1, vocab, dtype=np.float64)          # ids 1..vocab-1
        w = ranks ** (-s)
        self.cdf = np.cumsum(w / w.sum())
        self.cdf[-1] = 1.0

    def tokens(self, n: int) -> np.ndarray:
        return (np.searchsorted(self.cdf, self.rng.random(n), side="right") + 1).astype(np.int32)

    def docs(self, count: int) -> list:
        lens = self.rng.integers(self.lo, self.hi + 1, size=count)
        flat = self.tokens(int(lens.sum()))
        out, o = [], 0
        for n in lens:
            d = np.empty(n + 1, dtype=np.int32)
            d[0] = self.bos_id
            d[1:] = flat[o:o + n]
            out.append(d)
            o += n
        return out


class PackedRows:
    """Best-fit packer: yields int32 rows of ``row_len + 1`` tokens."""

    def __init__(self, source: ZipfDocs, row_len: int, buffer_docs: int = 512, rule=None, streams=None):
        self.src, self.row_len, self.buffer_docs = source, row_len, buffer_docs
        self.buf: list = []
        self.rule = rule                     # data.select.DocRule: documents it rejects never enter the buffer
        self.streams = streams               # data.streams.Streams: documents added after each refill, rows re-laid

    def _refill(self):
        while len(self.buf) < self.buffer_docs:
            docs = self.src.docs(self.buffer_docs)
            if self.rule is not None:
                docs = [d for d, keep in zip(docs, self.rule.decide(docs)) if keep]
            if self.streams is not None:
                docs = self.streams.after_refill(docs)
            self.buf.extend(docs)

    def next_row(self) -> np.ndarray:
        need = self.row_len + 1
        row = np.empty(need, dtype=np.int32)
        pos = 0
        while pos < need:
            self._refill()
            room = need - pos
            lens = np.fromiter((len(d) for d in self.buf), dtype=np.int64, count=len(self.buf))
            fits = np.nonzero(lens <= room)[0]
            if len(fits):
                i = int(fits[np.argmax(lens[fits])])          # the largest document that fits
                d = self.buf.pop(i)
                row[pos:pos + len(d)] = d
                pos += len(d)
            else:
                i = int(np.argmin(lens))                      # crop the shortest into the remaining room
                d = self.buf.pop(i)
                row[pos:] = d[:room]
                pos = need
        return self.streams.after_row(row) if self.streams is not None else row


def tail_marks(row: np.ndarray, bos_id: int, frac: float) -> np.ndarray:
    """Boolean mask over a packed row: the last ``frac`` of every document (its "answer span"; the synthetic stand-in
    for the reference's question-answer tails, ``QaPhase.spans`` round2/source/train.py:19717-19760)."""
    n = len(row)
    starts = np.flatnonzero(row == bos_id)
    if len(starts) == 0 or starts[0] != 0:
        starts = np.concatenate([[0], starts])
    ends = np.concatenate([starts[1:], [n]])
    doc = np.searchsorted(starts, np.arange(n), side="right") - 1
    length = (ends - starts)[doc]
    return (np.arange(n) - starts[doc]) >= np.ceil(length * (1.0 - frac))


def slice_windows(row: np.ndarray, seq_len: int, bos_id: int, mask_bos: bool = True, mark_tail: float = 0.0, vocab: int = 0):
    """One packed row -> ``(inputs [n, T] int32, targets [n, T] int64)``.  ``mark_tail > 0``: the targets inside the
    last ``mark_tail`` of each document are marked by adding ``vocab`` (the model weights their loss; reference:
    the loader's marks for ``qa_unmark``, round2/source/train.py:6504)."""
    n = (len(row) - 1) // seq_len
    trainable = None
    if (row < 0).any():                      # masked ids ride as -(id + 1) (data.streams.MaskedBlocks): never a target
        from .streams import decode_row
        row, trainable = decode_row(row)
    x = row[:n * seq_len].reshape(n, seq_len)
    y = row[1:n * seq_len + 1].astype(np.int64)
    if mask_bos:
        y = np.where(y == bos_id, -1, y)
    if trainable is not None:
        y = np.where(trainable[1:n * seq_len + 1], y, -1)
    if mark_tail > 0.0:
        marks = tail_marks(row, bos_id, mark_tail)[1:n * seq_len + 1]
        y = np.where(marks & (y >= 0), y + vocab, y)
    return x, y.reshape(n, seq_len)


class SynthLoader:
    """Per-rank loader.  ``next_step()`` returns pinned host tensors for one optimizer step on this rank:
    ``inputs [local_windows, T] int32`` and ``targets [local_windows, T] int64``."""

    def __init__(self, vocab: int, seq_len: int, local_windows: int, *, rank: int = 0, seed: int = 0,
                 doc_len=(128, 2048), zipf_s: float = 1.1, bos_id: int = 0, pin: bool = False, rule=None,
                 shard_of: int = 0, streams=None):
        # shard_of = W > 0: every rank draws the same stream (the seed alone decides it), packs the whole job's step and
        # keeps windows rank, rank + W, ...: the global batch of a step is then the same set of windows at any rank
        # count, which makes losses comparable across 1, 2, 4 and 8 ranks.  0: one independent stream per rank.
        self.seq_len, self.local_windows, self.bos_id, self.vocab = seq_len, local_windows, bos_id, vocab
        self.mark_tail = 0.0                 # > 0: answer-span marks on the targets (set when the answer phase starts)
        self.shard_of, self.rank = int(shard_of), rank
        self.docs = ZipfDocs(vocab, zipf_s, doc_len, seed=seed * 1000003 + (0 if shard_of else rank), bos_id=bos_id)
        self.rule, self.streams = rule, streams
        self.rows = PackedRows(self.docs, seq_len * local_windows * max(1, self.shard_of), rule=rule, streams=streams)
        self.pin = pin and torch.cuda.is_available()
        self.epoch = 0

    def next_step(self):
        if self.streams is not None:
            self.streams.begin_batch(self.epoch)
        row = self.rows.next_row()
        if self.streams is not None:
            self.streams.end_batch()
        self.epoch += 1
        x, y = slice_windows(row, self.seq_len, self.bos_id, mark_tail=self.mark_tail, vocab=self.vocab)
        if self.shard_of:
            x, y = x[self.rank::self.shard_of], y[self.rank::self.shard_of]
        xt, yt = torch.from_numpy(np.ascontiguousarray(x)), torch.from_numpy(np.ascontiguousarray(y))
        if self.pin:
            xt, yt = xt.pin_memory(), yt.pin_memory()
        return xt, yt

    def set_seq_len(self, seq_len: int):
        """Sequence ramp: same tokens per step in shorter windows (reference: ``SeqRamp``,
        round2/source/train.py:21228-21311)."""
        tokens = self.seq_len * self.local_windows
        if tokens % seq_len:
            raise ValueError("step tokens must be a multiple of the new window length")
        self.seq_len, self.local_windows = seq_len, tokens // seq_len


class Prefetcher:
    """Host worker that prepares step s+1 while step s runs on the device, with double buffers so that a buffer is
    rewritten only after the step that last read it has been handed back (reference: ``LoaderPrefetchT2``,
    round2/source/train.py:13866-13932).  Exceptions in the worker are re-raised on the caller's thread."""

    def __init__(self, fn):
        self.fn = fn
        self._thr = None
        self._out = None
        self._exc = None

    def start(self):
        if self._thr is not None:
            raise RuntimeError("prefetch already in flight")
        self._out, self._exc = None, None

        def work():
            try:
                self._out = self.fn()
            except BaseException as exc:  # noqa: BLE001 - surfaced by finish()
                self._exc = exc

        self._thr = threading.Thread(target=work, daemon=True)
        self._thr.start()

    def finish(self):
        if self._thr is None:
            self.start()
        self._thr.join()
        self._thr = None
        if self._exc is not None:
            raise self._exc
        return self._out


def bytes_per_token_table(vocab: int, seed: int = 0) -> torch.Tensor:
    """Fixed synthetic ``bytes per token`` table for bits-per-byte evaluation: frequent tokens are short
    (1-2 bytes), rare tokens long; BOS counts zero bytes."""
    rng = np.random.default_rng(seed)
    ranks = np.arange(vocab)
    base = 1 + np.minimum(7, np.log2(1 + ranks).astype(np.int64) // 2)
    jitter = rng.integers(0, 2, size=vocab)
    b = (base + jitter).astype(np.int64)
    b[0] = 0
    return torch.from_numpy(b)
