"""Document streams that ride on the packer: what enters the buffer besides the source's documents, and how a packed
row is laid out.  Token-id forms of the reference's loader lanes (which read text through the tokenizer; a synthetic
stream has ids only, so every criterion here is a function of ids, lengths and hashes):

* ``PoolMix`` -- a stored pool of documents mixed in at a token share from a decision point on, each document at most
  ``rep`` times, this rank's documents by hash, paid from a token debt (reference: ``DselStream``,
  round2/source/train.py:18841-18940).
* ``StrataMix`` -- representatives added from the stratum (class x length bucket) whose token share has fallen furthest
  below its share in the first phase (reference: ``CovselRule``, round2/source/train.py:19584-19690).
* ``MaskedBlocks`` -- blocks of examples cut from the refill's own documents (context masked, continuation trained),
  masked ids carried as ``-(id + 1)`` until the row is sliced, at a share of the tokens entering the buffer with the
  late schedule (reference: ``RelayStream``, round2/source/train.py:16386-16420).
* ``EdgeRelay`` -- a packed row re-laid from its own pieces, each piece whole and in its own order, so that fewer
  pieces are cut by a window edge (reference: ``EdgeRelay``, round2/source/train.py:17953-18090).
* ``SharedDedup`` -- duplicate removal across ranks through a bloom filter and per-batch slot files in a shared
  directory, merged by rank 0 (reference: ``DedupRider``, round2/source/train.py:18093-18290).

``Streams.parse`` builds them from one switch string; ``PackedRows`` calls ``after_refill`` on every refill's kept
documents and ``after_row`` on every packed row; ``decode_row`` turns the masked encoding into ids and a trainable mask.
"""
from __future__ import annotations

import hashlib
import os
import time

import numpy as np

def doc_hash(ids: np.ndarray, seed: int = 0) -> int:
    """64-bit hash of a document's ids (masked ids count as the ids they stand for)."""
    a = np.ascontiguousarray(ids, dtype=np.int64)
    if len(a) and a.min() < 0:
        a = np.where(a < 0, -a - 1, a)
    key = int(seed & 0xFFFFFFFFFFFFFFFF).to_bytes(8, "little")
    return int.from_bytes(hashlib.blake2b(a.astype(np.uint32).tobytes(), digest_size=8, key=key).digest(), "little")


class _Debt:
    """Token debt of an added stream: every refill's own tokens add ``share / (1 - share)`` of themselves, every added
    document takes its tokens off, so the stream's tokens are ``share`` of all tokens since the stream was switched on."""

    def __init__(self, share: float):
        if not 0.0 <= share < 1.0:
            raise ValueError(f"a stream's token share must be in [0, 1), got {share}")
        self.share, self.debt, self.base_tokens, self.added_tokens = share, 0.0, 0, 0

    def earn(self, tokens: int, factor: float = 1.0):
        self.base_tokens += tokens
        s = min(0.95, self.share * factor)
        self.debt += tokens * s / (1.0 - s)

    def pay(self, tokens: int):
        self.debt -= tokens
        self.added_tokens += tokens


class PoolMix:
    def __init__(self, pool: list, *, share: float, start: float = 0.0, rep: int = 1, rank: int = 0, world: int = 1,
                 seed: int = 0):
        self.pool, self.start, self.rep, self.seed = pool, start, max(1, rep), seed
        self.mine = [i for i, d in enumerate(pool) if doc_hash(d, seed) % world == rank]
        self.debt = _Debt(share)
        self.phase, self.active = 0.0, False
        self.passes, self.next, self.order = 0, 0, []
        self.count = dict(docs=0, tokens=0, short=0, calls=0)

    def _begin_pass(self):
        # an order of its own per pass: ascending hash of the document's number mixed with the pass
        keys = [doc_hash(np.asarray([i, self.passes], dtype=np.uint32), self.seed) for i in self.mine]
        self.order = [i for _, i in sorted(zip(keys, self.mine))]
        self.next = 0

    def mix(self, docs: list) -> list:
        """The refill's documents followed by this rank's pool documents while the debt is positive."""
        self.count["calls"] += 1
        if not self.active:
            if self.phase < self.start:
                return docs
            self.active = True
            self._begin_pass()
        self.debt.earn(sum(len(d) for d in docs))
        out = list(docs)
        while self.debt.debt > 0:
            if self.next >= len(self.order):
                self.passes += 1
                if self.passes >= self.rep or not self.mine:
                    self.count["short"] += 1              # the passes are spent: this refill adds nothing more
                    break
                self._begin_pass()
            d = self.pool[self.order[self.next]]
            self.next += 1
            out.append(d)
            self.debt.pay(len(d))
            self.count["docs"] += 1
            self.count["tokens"] += len(d)
        return out

    def line(self) -> str:
        c = self.count
        got = self.debt.added_tokens / max(1, self.debt.added_tokens + self.debt.base_tokens)
        return (f"pool mix: {c['docs']} documents / {c['tokens']} tokens added in {c['calls']} refills "
                f"(share {got:.4f} of {self.debt.share:g}), pass {self.passes + 1} of {self.rep}, short {c['short']}")


LENGTH_EDGES = (64, 128, 256, 512, 1024)            # six length buckets


def length_bucket(n: int) -> int:
    return int(np.searchsorted(LENGTH_EDGES, n, side="right"))


class StrataMix:
    """Two classes (does the document lean to frequent or to rare ids: its median id against ``split``) x six length
    buckets = 12 strata.  Until the decision (``phase < start``) the token share of every stratum is recorded; from then
    on representatives are added, always from the stratum furthest below its recorded share whose queue holds one."""

    def __init__(self, pool: list, *, share: float, start: float, split: int, rank: int = 0, world: int = 1, seed: int = 0):
        self.ns = 2 * (len(LENGTH_EDGES) + 1)
        self.split, self.start = split, start
        self.queues = [[] for _ in range(self.ns)]
        for d in pool:                                           # best first: the pool's own order
            if doc_hash(d, seed) % world == rank:
                self.queues[self.stratum(d)].append(d)
        self.heads = [0] * self.ns
        self.p1 = np.zeros(self.ns)                              # phase 1's tokens per stratum
        self.seen = np.zeros(self.ns)                            # tokens per stratum since the decision (kit + added)
        self.debt = _Debt(share)
        self.phase, self.active = 0.0, False
        self.rep = np.zeros((2, self.ns), dtype=np.int64)       # [documents added, tokens added][stratum]
        self.short = 0

    def stratum(self, d: np.ndarray) -> int:
        body = d[1:] if len(d) > 1 else d
        cls = int(np.median(body) > self.split)
        return cls * (self.ns // 2) + length_bucket(len(body))

    def mix(self, docs: list) -> list:
        if not self.active and self.phase < self.start:
            for d in docs:
                self.p1[self.stratum(d)] += len(d)
            return docs
        self.active = True
        target = self.p1 / max(1.0, self.p1.sum())
        for d in docs:
            self.seen[self.stratum(d)] += len(d)
        self.debt.earn(sum(len(d) for d in docs))
        out = list(docs)
        while self.debt.debt > 0:
            live = [s for s in range(self.ns) if self.heads[s] < len(self.queues[s])]
            if not live:
                self.short += 1
                break
            gap = target - self.seen / max(1.0, self.seen.sum())
            s = max(live, key=lambda k: gap[k])
            d = self.queues[s][self.heads[s]]
            self.heads[s] += 1
            out.append(d)
            self.debt.pay(len(d))
            self.seen[s] += len(d)
            self.rep[0, s] += 1
            self.rep[1, s] += len(d)
        return out

    def line(self) -> str:
        return (f"strata mix: {int(self.rep[0].sum())} representatives / {int(self.rep[1].sum())} tokens added over "
                f"{int((self.rep[0] > 0).sum())} of {self.ns} strata, short {self.short}")


class MaskedBlocks:
    """Blocks of ``examples`` examples, each cut from one of the refill's documents: a context span (masked), the
    separator id (masked) and the span that follows it in the document (trained).  A block is BOS followed by its
    examples; masked ids are carried as ``-(id + 1)``."""

    def __init__(self, *, share: float, sep_id: int, bos_id: int = 0, examples: int = 4, context: int = 24, answer: int = 8,
                 late: bool = False, seed: int = 0):
        self.debt = _Debt(share)
        self.sep_id, self.bos_id, self.examples, self.context, self.answer = sep_id, bos_id, examples, context, answer
        self.late, self.phase = late, 0.0
        self.rng = np.random.default_rng(seed)
        self.count = dict(blocks=0, examples=0, tokens=0, masked=0)

    def _example(self, d: np.ndarray):
        need = self.context + self.answer
        if len(d) - 1 < need:
            return None
        o = 1 + int(self.rng.integers(0, len(d) - need))
        ctx, ans = d[o:o + self.context].astype(np.int64), d[o + self.context:o + need].astype(np.int64)
        return np.concatenate([-(ctx + 1), [-(self.sep_id + 1)], ans])

    def make(self, docs: list) -> list:
        """Blocks for one refill (possibly none), made only of the refill's own documents."""
        factor = (0.75 if self.phase < 0.8 else 2.0) if self.late else 1.0
        self.debt.earn(sum(len(d) for d in docs), factor)
        out = []
        cands = [d for d in docs if len(d) - 1 >= self.context + self.answer]
        while self.debt.debt > 0 and cands:
            parts = [np.asarray([self.bos_id], dtype=np.int64)]
            for _ in range(self.examples):
                ex = self._example(cands[int(self.rng.integers(0, len(cands)))])
                parts.append(ex)
            blk = np.concatenate(parts)
            out.append(blk)
            self.debt.pay(len(blk))
            self.count["blocks"] += 1
            self.count["examples"] += self.examples
            self.count["tokens"] += len(blk)
            self.count["masked"] += int((blk < 0).sum())
        return out

    def line(self) -> str:
        c = self.count
        return f"masked blocks: {c['blocks']} blocks / {c['examples']} examples / {c['tokens']} tokens ({c['masked']} masked)"


def decode_row(row: np.ndarray):
    """Packed row with masked ids as ``-(id + 1)`` -> ``(ids int32, trainable bool)``."""
    neg = row < 0
    if not neg.any():
        return row.astype(np.int32, copy=False), np.ones(len(row), dtype=bool)
    ids = np.where(neg, -row - 1, row).astype(np.int32)
    return ids, ~neg


class EdgeRelay:
    """Re-lays a packed row of windows of ``window`` tokens from its own pieces.  A piece runs from one BOS to the next
    (the row's leading fragment, if it does not start with BOS, and the cropped last piece stay where they are); its
    kind is a block if it holds a masked id, else a plain document.  Pieces keep their tokens and inner order; only
    their order in the row changes.  Nearly every window edge has to cut some piece (the lengths do not add up to whole
    windows), so the re-lay chooses which: each window is filled with pieces that fit its room whole, blocks first, and
    when nothing fits the longest remaining plain document is laid across the edge, where a cut costs the smallest
    share of a piece's context.  A row is re-laid only if that cuts fewer blocks, or as many blocks and fewer short
    pieces (under half a window).  Counters: rows, rows re-laid, pieces, pieces longer than a window, and the pieces
    cut by an edge by kind (plain, short plain, block) before and after."""

    KEYS = ("rows", "moved", "pieces", "long")

    def __init__(self, window: int, bos_id: int = 0):
        self.w, self.bos = window, bos_id
        self.n = dict.fromkeys(self.KEYS, 0)
        self.split = {"before": [0, 0, 0], "after": [0, 0, 0]}     # plain, short plain, block
        self.seconds = 0.0

    def _cuts(self, lengths, kinds, pos: int):
        out = [0, 0, 0]
        for n, k in zip(lengths, kinds):
            if n and pos // self.w != (pos + n - 1) // self.w:
                out[2 if k else (1 if n < self.w // 2 else 0)] += 1
            pos += n
        return out

    def relay(self, row: np.ndarray) -> np.ndarray:
        t0 = time.perf_counter()
        ids = np.where(row < 0, -row - 1, row) if (row < 0).any() else row
        starts = np.flatnonzero(ids == self.bos)
        self.n["rows"] += 1
        if len(starts) < 3:
            return row
        head = row[:starts[0]]
        cuts = list(starts) + [len(row)]
        pieces = [row[cuts[i]:cuts[i + 1]] for i in range(len(starts))]
        last = pieces.pop()                                      # possibly cropped: it stays at the row's end
        lengths = [len(p) for p in pieces]
        kinds = [int(p.min() < 0) for p in pieces]
        before = self._cuts(lengths, kinds, len(head))
        order, pos = [], len(head)
        left = sorted(range(len(pieces)), key=lambda i: (-kinds[i], -lengths[i]))      # blocks first, then by length
        while left:
            room = self.w - pos % self.w
            pick = next((i for i in left if lengths[i] <= room), None)
            if pick is None:                                     # something has to cross the edge: the longest plain piece
                plain = [i for i in left if not kinds[i]]
                pick = max(plain or left, key=lambda i: lengths[i])
            left.remove(pick)
            order.append(pick)
            pos += lengths[pick]
        after = self._cuts([lengths[i] for i in order], [kinds[i] for i in order], len(head))
        self.n["pieces"] += len(pieces) + 1
        self.n["long"] += sum(1 for n in lengths if n > self.w)
        better = (after[2], after[1]) < (before[2], before[1])
        for k in range(3):
            self.split["before"][k] += before[k]
            self.split["after"][k] += (after if better else before)[k]
        if not better:
            self.seconds += time.perf_counter() - t0
            return row
        self.n["moved"] += 1
        out = np.concatenate([head] + [pieces[i] for i in order] + [last]).astype(row.dtype, copy=False)
        self.seconds += time.perf_counter() - t0
        return out

    def line(self) -> str:
        n = self.n
        return (f"edge relay: {n['rows']} rows, {n['moved']} re-laid, {n['pieces']} pieces ({n['long']} longer than a window); "
                f"pieces cut by an edge [plain, short plain, block] {self.split['before']} -> {self.split['after']}; "
                f"{self.seconds:.2f} s")


class SharedDedup:
    """Duplicate removal across ranks.  Files under ``root``: ``bloom`` (the filter, memory-mapped by every rank),
    ``merged`` (the latest batch rank 0 has folded in) and ``slot_<b>_<r>.npy`` (the hashes rank r accepted in batch b).
    ``begin_batch(b)``: rank 0 waits (bounded) for every rank's slot of batch ``b - lag``, folds them into the filter and
    publishes ``merged``; the others wait (bounded) until ``merged >= b - lag``, so what a rank sees in batch b does not
    depend on timing.  ``decide`` drops a document whose hash is in the filter or was accepted earlier on this rank;
    ``end_batch`` writes this rank's slot."""

    def __init__(self, root: str, rank: int, world: int, bits: int = 24, lag: int = 2, wait_s: float = 30.0, seed: int = 0):
        self.root, self.rank, self.world, self.bits, self.lag, self.wait_s, self.seed = root, rank, world, bits, lag, wait_s, seed
        self.batch, self.pending, self.local = -1, [], set()
        self.n = dict(read=0, dropped_filter=0, dropped_local=0, merged_hashes=0, waits=0)
        nbytes = (1 << bits) // 8
        path = os.path.join(root, "bloom")
        if rank == 0:
            os.makedirs(root, exist_ok=True)
            if not os.path.exists(path):
                tmp = path + f".tmp{os.getpid()}"
                with open(tmp, "wb") as fh:
                    fh.truncate(nbytes)
                os.replace(tmp, path)
            self._put_merged(-1)
        self._wait(lambda: os.path.exists(path) and os.path.exists(os.path.join(root, "merged")), "the filter file")
        self.bloom = np.memmap(path, dtype=np.uint8, mode="r+" if rank == 0 else "r", shape=(nbytes,))

    # -- files ---------------------------------------------------------------------------------------------------
    def _wait(self, ready, what: str):
        t0 = time.time()
        while not ready():
            if time.time() - t0 > self.wait_s:
                raise TimeoutError(f"shared dedup: rank {self.rank} waited {self.wait_s:.0f} s for {what}")
            self.n["waits"] += 1
            time.sleep(0.005)

    def _put_merged(self, b: int):
        tmp = os.path.join(self.root, f"merged.tmp{os.getpid()}")
        with open(tmp, "w") as fh:
            fh.write(str(b))
        os.replace(tmp, os.path.join(self.root, "merged"))

    def _merged(self) -> int:
        try:
            with open(os.path.join(self.root, "merged")) as fh:
                return int(fh.read().strip() or -1)
        except (OSError, ValueError):
            return -2

    def _slot(self, b: int, r: int) -> str:
        return os.path.join(self.root, f"slot_{b}_{r}.npy")

    def _bits_of(self, h: np.ndarray):
        mask = np.uint64((1 << self.bits) - 1)
        return [(h >> np.uint64(s)) & mask for s in (0, 20, 40)]

    # -- batches -------------------------------------------------------------------------------------------------
    def begin_batch(self, b: int):
        self.batch = b
        due = b - self.lag
        if due < 0:
            return
        if self.rank == 0:
            for bb in range(max(0, self._merged() + 1), due + 1):
                for r in range(self.world):
                    self._wait(lambda: os.path.exists(self._slot(bb, r)), f"rank {r}'s slot of batch {bb}")
                    h = np.load(self._slot(bb, r))
                    for idx in self._bits_of(h):
                        np.bitwise_or.at(self.bloom, (idx >> np.uint64(3)).astype(np.int64),
                                         (np.uint8(1) << (idx & np.uint64(7)).astype(np.uint8)))
                    self.n["merged_hashes"] += len(h)
                    os.remove(self._slot(bb, r))
                self.bloom.flush()
                self._put_merged(bb)
        else:
            self._wait(lambda: self._merged() >= due, f"the merge of batch {due}")

    def decide(self, docs: list) -> list:
        keep = []
        for d in docs:
            self.n["read"] += 1
            h = np.uint64(doc_hash(d, self.seed))
            if int(h) in self.local:
                self.n["dropped_local"] += 1
                keep.append(False)
                continue
            hit = all(self.bloom[int(i[0]) >> 3] & (1 << (int(i[0]) & 7)) for i in self._bits_of(np.asarray([h], dtype=np.uint64)))
            if hit:
                self.n["dropped_filter"] += 1
                keep.append(False)
                continue
            self.local.add(int(h))
            self.pending.append(int(h))
            keep.append(True)
        return keep

    def end_batch(self):
        tmp = self._slot(self.batch, self.rank) + ".tmp.npy"
        np.save(tmp, np.asarray(self.pending, dtype=np.uint64))
        os.replace(tmp, self._slot(self.batch, self.rank))
        self.pending = []

    def line(self) -> str:
        n = self.n
        return (f"shared dedup: {n['read']} documents read, dropped {n['dropped_filter']} by the filter and "
                f"{n['dropped_local']} by this rank's own set; rank 0 folded {n['merged_hashes']} hashes")


class Streams:
    """The packer's riders, in the reference's order: the cross-rank dedup decides on the source's documents, the pool
    and the strata add theirs, the masked blocks are cut from what the refill then holds, and every packed row is re-laid."""

    def __init__(self, dedup=None, pool=None, strata=None, blocks=None, edge=None):
        self.dedup, self.pool, self.strata, self.blocks, self.edge = dedup, pool, strata, blocks, edge

    @classmethod
    def parse(cls, spec: str, *, vocab: int, seq_len: int, bos_id: int = 0, rank: int = 0, world: int = 1, seed: int = 0,
              pool_docs=None):
        """``"pool:0.1@0.3x2,strata:0.05@0.3,blocks:0.02+late,edge,dedup:/path"`` (empty string: nothing).  ``pool`` and
        ``strata`` draw from ``pool_docs`` (a list of id arrays; default: 2048 documents from a Zipf source of their own)."""
        if not spec:
            return None
        kw = {}
        store = pool_docs

        def pool_store():
            nonlocal store
            if store is None:
                from .synth import ZipfDocs
                store = ZipfDocs(vocab, seed=seed * 7919 + 17, bos_id=bos_id).docs(2048)
            return store

        for part in spec.split(","):
            key, _, val = part.strip().partition(":")
            if key == "pool":
                share, _, rest = val.partition("@")
                start, _, rep = rest.partition("x")
                kw["pool"] = PoolMix(pool_store(), share=float(share), start=float(start or 0), rep=int(rep or 1), rank=rank,
                                     world=world, seed=seed)
            elif key == "strata":
                share, _, start = val.partition("@")
                kw["strata"] = StrataMix(pool_store(), share=float(share), start=float(start or 0), split=max(2, vocab // 64),
                                         rank=rank, world=world, seed=seed)
            elif key == "blocks":
                share, _, flag = val.partition("+")
                kw["blocks"] = MaskedBlocks(share=float(share), sep_id=vocab - 1, bos_id=bos_id, late=flag == "late",
                                            seed=seed * 31 + rank)
            elif key == "edge":
                kw["edge"] = EdgeRelay(seq_len, bos_id)
            elif key == "dedup":
                kw["dedup"] = SharedDedup(val, rank, world, seed=seed)
            else:
                raise ValueError(f"data streams: unknown field {key!r} in {spec!r}")
        return cls(**kw)

    def set_phase(self, phase: float):
        for s in (self.pool, self.strata, self.blocks):
            if s is not None:
                s.phase = phase

    def begin_batch(self, b: int):
        if self.dedup is not None:
            self.dedup.begin_batch(b)

    def end_batch(self):
        if self.dedup is not None:
            self.dedup.end_batch()

    def after_refill(self, docs: list) -> list:
        if self.dedup is not None:
            docs = [d for d, keep in zip(docs, self.dedup.decide(docs)) if keep]
        if self.pool is not None:
            docs = self.pool.mix(docs)
        if self.strata is not None:
            docs = self.strata.mix(docs)
        if self.blocks is not None:
            docs = docs + self.blocks.make(docs)
        return docs

    def after_row(self, row: np.ndarray) -> np.ndarray:
        return self.edge.relay(row) if self.edge is not None else row

    def lines(self) -> list:
        return [s.line() for s in (self.dedup, self.pool, self.strata, self.blocks, self.edge) if s is not None]
