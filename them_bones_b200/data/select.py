"""Document selection on token ids, applied while the packer's buffer is refilled.

The reference's selection rules (``DataRule``, round2/source/train.py:14526-14800) score real text with tokenizer-derived
tables; a synthetic token stream has no text, so the rules that need only token ids are built here:

* a **length floor / ceiling**;
* the **typicality band** (the reference's rule 3): every document gets the mean log-probability of its tokens under a
  running hashed-bigram model with unigram back-off that is updated with every document read; after a warm-up, a
  document is kept only if its score lies inside a quantile band of the scores of the last ``RING`` documents (too
  predictable = boilerplate, too surprising = noise);
* **near-duplicate removal**: a document whose leading ``dedup_prefix`` tokens were seen before is dropped;
* a **start phase**: the rule acts only once the run's elapsed fraction has reached ``start`` (set ``phase`` before each
  refill), and counters are kept per phase, as in the reference.

``decide(docs)`` returns the keep flags; ``PackedRows`` drops the rest before they enter the buffer.
"""
from __future__ import annotations

import numpy as np


class DocRule:
    RING = 65536            # the band's quantiles are over the last RING scored documents
    HASH_BITS = 22          # buckets of the hashed bigram counts

    def __init__(self, vocab: int, *, min_len: int = 0, max_len: int = 0, band=(0.0, 1.0), warm: int = 1024,
                 dedup_prefix: int = 0, start: float = 0.0, bos_id: int = 0):
        self.vocab, self.bos_id = vocab, bos_id
        self.min_len, self.max_len = min_len, max_len
        self.band, self.warm, self.dedup_prefix, self.start = tuple(band), warm, dedup_prefix, start
        self.phase = 0.0
        self.use_band = self.band != (0.0, 1.0)
        if self.use_band:
            self.bigram = np.zeros(1 << self.HASH_BITS, dtype=np.int32)
            self.context = np.zeros(vocab, dtype=np.int64)
            self.unigram = np.ones(vocab, dtype=np.int64)
            self.total = vocab
            self.ring = np.zeros(self.RING, dtype=np.float64)
            self.scored = 0
        self.seen = set()
        self.count = {k: np.zeros(2, dtype=np.int64) for k in
                      ("docs_read", "docs_kept", "drop_length", "drop_band", "drop_dup", "tokens_read", "tokens_kept")}

    @classmethod
    def parse(cls, spec: str, vocab: int, bos_id: int = 0):
        """``"len:64-4096,band:0.05-0.95,warm:512,dedup:32,from:0.1"`` -> rule (empty string: no rule)."""
        if not spec:
            return None
        kw = {}
        for part in spec.split(","):
            key, _, val = part.strip().partition(":")
            if key == "len":
                lo, _, hi = val.partition("-")
                kw["min_len"], kw["max_len"] = int(lo or 0), int(hi or 0)
            elif key == "band":
                lo, _, hi = val.partition("-")
                kw["band"] = (float(lo), float(hi))
            elif key == "warm":
                kw["warm"] = int(val)
            elif key == "dedup":
                kw["dedup_prefix"] = int(val)
            elif key == "from":
                kw["start"] = float(val)
            else:
                raise ValueError(f"data rule: unknown field {key!r} in {spec!r}")
        return cls(vocab, bos_id=bos_id, **kw)

    # ------------------------------------------------------------------------------------------------------------
    def _bucket(self, a: np.ndarray, b: np.ndarray) -> np.ndarray:
        h = (a.astype(np.uint64) * np.uint64(0x9E3779B97F4A7C15) + b.astype(np.uint64) * np.uint64(0xC2B2AE3D27D4EB4F))
        return (h >> np.uint64(64 - self.HASH_BITS)).astype(np.int64)

    def score(self, ids: np.ndarray) -> float:
        """Mean log-probability per token under the running model (bigram with add-one unigram back-off), then the
        model learns the document."""
        if len(ids) < 2:
            return 0.0
        a, b = ids[:-1].astype(np.int64), ids[1:].astype(np.int64)
        bk = self._bucket(a, b)
        uni = self.unigram[b] / self.total
        p = (self.bigram[bk] + uni) / (self.context[a] + 1.0)
        s = float(np.log(np.minimum(p, 1.0)).mean())
        np.add.at(self.bigram, bk, 1)
        np.add.at(self.context, a, 1)
        np.add.at(self.unigram, ids.astype(np.int64), 1)
        self.total += len(ids)
        return s

    def decide(self, docs: list) -> list:
        """Keep flag per document (each starts with BOS, which no feature reads)."""
        live = int(self.phase >= self.start)
        keep = []
        for d in docs:
            ids = d[1:] if len(d) and d[0] == self.bos_id else d
            n = len(ids)
            self.count["docs_read"][live] += 1
            self.count["tokens_read"][live] += len(d)
            ok = True
            reason = None
            if self.use_band:                                   # the model reads every document, kept or not
                s = self.score(ids)
                self.ring[self.scored % self.RING] = s
                self.scored += 1
            if live:
                if (self.min_len and n < self.min_len) or (self.max_len and n > self.max_len):
                    ok, reason = False, "drop_length"
                elif self.use_band and self.scored > self.warm:
                    window = self.ring[:min(self.scored, self.RING)]
                    lo, hi = np.quantile(window, self.band)
                    if not lo <= s <= hi:
                        ok, reason = False, "drop_band"
                if ok and self.dedup_prefix:
                    key = ids[:self.dedup_prefix].tobytes()
                    if key in self.seen:
                        ok, reason = False, "drop_dup"
                    else:
                        self.seen.add(key)
            if ok:
                self.count["docs_kept"][live] += 1
                self.count["tokens_kept"][live] += len(d)
            else:
                self.count[reason][live] += 1
            keep.append(ok)
        return keep

    def line(self) -> str:
        c = self.count
        return ("data rule: read %d docs / %d tokens, kept %d / %d; dropped length %d, band %d, duplicate %d" %
                (int(c["docs_read"].sum()), int(c["tokens_read"].sum()), int(c["docs_kept"].sum()), int(c["tokens_kept"].sum()),
                 int(c["drop_length"].sum()), int(c["drop_band"].sum()), int(c["drop_dup"].sum())))
