"""Gradient-trained hashed n-gram lookup tables, row-sharded over the data-parallel ranks' HBM.

Role in the model: for every position the previous ``order`` token ids are hashed to a row of a ``[rows, n_embd]``
table and the row is added to the residual stream at the input (one table per order, e.g. bigram and trigram).  The
reference keeps its n-gram table in host shared memory and exchanges sparse gradients through staging files and
barriers (``NgramHostTable``, round2/source/train.py:3526-3862: ``ids`` 3621, ``gather`` 3627, ``_exchange`` 3653,
``step`` 3678); kept from it: zero initialisation (the first forward equals the table-free model), causal hashing with
a pad id before the window start, owner-computes updates (owner = ``row % world``), gradients of duplicate rows summed
then averaged over ranks, its row-wise RMS update with one fp32 second moment per row, stochastic rounding of updated
rows to bf16, and no update from a non-finite gradient.  Not kept: the one-step-stale application (``NgramStaleT21``,
:13934), which exists to hide the host table's update behind a worker thread; the device update here takes
milliseconds and is applied in step.

Here each rank owns ``rows / world`` rows in device memory.  Two transports (``exchange``):

* the peer-memory one (``parallel.symm.PeerTableExchange``, GPUs): lookups read the owners' shards through NVLink peer
  pointers; gradient rows are pushed into the owner's staging buffer from inside backward, and the owner's update
  (``csrc/tables.cu``) sums duplicates in sorted order and writes the table in place -- no library collective, no host
  synchronisation anywhere in a step;
* ``parallel.table_a2a.CollectiveExchange`` (NCCL / gloo all-to-all; CPU path, baseline and oracle), whose update is
  the PyTorch statement of the same arithmetic.

Optimizer state (``opt``): ``"rowrms"`` keeps one fp32 second moment per row (4 bytes per row: 2^26 rows x 2 tables over
8 ranks is 67 MB per rank); ``"adam"`` keeps dense fp32 first and second moments (8 bytes per element: the same tables
would need 1.4 TB), on the device or, with ``host_state``, in pinned host memory streamed on a side stream.  ``"auto"``
takes Adam while its moments fit in a quarter of the device and the row-wise form beyond that.
"""
from __future__ import annotations

import torch

from ..ref import functional as RF


class _LookupFn(torch.autograd.Function):
    """Forward: rows gathered from the sharded table.  Backward: hands ``d rows`` to the table object (no dense
    gradient is ever formed)."""

    @staticmethod
    def forward(ctx, anchor, tables, order_slot, ids):
        ctx.tables, ctx.order_slot = tables, order_slot
        ctx.save_for_backward(ids)
        return tables.gather(order_slot, ids)

    @staticmethod
    def backward(ctx, g):
        (ids,) = ctx.saved_tensors
        ctx.tables.record_grad(ctx.order_slot, ids, g)
        return torch.zeros(()), None, None, None


class HashedTables:
    def __init__(self, orders, rows: int, dim: int, *, seed: int = 0, device="cpu", dtype=torch.float32,
                 group=None, world: int = 1, rank: int = 0, host_state: bool = False,
                 betas=(0.9, 0.99), eps: float = 1e-8, decay: float = 0.0, exchange=None, bits: int = 0, opt: str = "auto"):
        if rows % world:
            raise ValueError("table rows must divide over the ranks")
        if opt not in ("auto", "adam", "rowrms"):
            raise ValueError(f"table optimizer {opt!r}: expected auto, adam or rowrms")
        self.orders, self.rows, self.dim, self.seed = tuple(orders), rows, dim, seed
        self.group, self.world, self.rank = group, world, rank
        self.device, self.dtype = torch.device(device), dtype
        # bits 1 / 4: every read (training and scoring alike) takes the row's packed view, the gradient goes straight
        # through to the master row, and the checkpoint stores the view (reference: R2_NGRAM_BITS,
        # round2/source/train.py:1016-1029).  rows_are_views: the shards were loaded from such a checkpoint.
        self.bits, self.rows_are_views = bits, False
        self.local_rows = rows // world
        self.shards = [torch.zeros(self.local_rows, dim, dtype=dtype, device=self.device) for _ in self.orders]
        dense_state = 2 * 4 * self.local_rows * dim * len(self.orders)
        have = torch.cuda.get_device_properties(self.device).total_memory if self.device.type == "cuda" else 0
        if opt == "auto":
            opt = "adam" if (self.device.type != "cuda" or dense_state <= 0.25 * have or host_state is True) else "rowrms"
        self.opt = opt
        self.host_state = False
        self.exp_avg, self.exp_avg_sq, self.row_sq = [], [], []
        if opt == "adam":
            # dense moments: on the device while they fit, else (or on request) in pinned host memory, streamed per step;
            # the host route pays a CPU gather / scatter of every touched row and is for tables the GPU cannot hold
            if host_state == "auto":
                host_state = self.device.type == "cuda" and dense_state > 0.35 * have
            self.host_state = bool(host_state) and self.device.type == "cuda"
            sdev = "cpu" if self.host_state else self.device
            mk = lambda: torch.zeros(self.local_rows, dim, dtype=torch.float32, device=sdev)  # noqa: E731
            self.exp_avg = [mk() for _ in self.orders]
            self.exp_avg_sq = [mk() for _ in self.orders]
            if self.host_state:
                self.exp_avg = [t.pin_memory() for t in self.exp_avg]
                self.exp_avg_sq = [t.pin_memory() for t in self.exp_avg_sq]
                self.side_stream = torch.cuda.Stream(device=self.device)
        else:
            self.row_sq = [torch.zeros(self.local_rows, dtype=torch.float32, device=self.device) for _ in self.orders]
        self.betas, self.eps, self.decay = betas, eps, decay
        self.steps = 0
        self.pending = []           # [(order_slot, ids [n], grads [n, dim])] recorded by backward
        self._anchor = torch.zeros((), requires_grad=True)
        from ..parallel import table_a2a
        self.exchange = exchange or table_a2a.make_exchange(group, world, rank, self.device)
        self.stats = dict(updates=0, skipped=0, touched=0)

    def state_bytes(self) -> dict:
        """Bytes this rank holds: table shards and optimizer state (device or pinned host)."""
        shards = sum(t.numel() * t.element_size() for t in self.shards)
        state = sum(t.numel() * t.element_size() for t in self.exp_avg + self.exp_avg_sq + self.row_sq)
        return dict(shards=shards, state=state, state_on_host=self.host_state, opt=self.opt)

    # -- hashing / lookup -----------------------------------------------------------------------------------
    def ids(self, idx: torch.Tensor, doc_start=None):
        """``[len(orders), B, T]`` int64 row ids."""
        return torch.stack([RF.ngram_rows(idx, o, self.rows, self.seed + j, doc_start)
                            for j, o in enumerate(self.orders)])

    def owner_local(self, ids):
        return ids % self.world, ids // self.world

    def gather(self, order_slot: int, ids: torch.Tensor) -> torch.Tensor:
        """Rows for global ids ``[n]`` -> ``[n, dim]`` (all-to-all with the owners when sharded)."""
        rows = self.exchange.lookup(self.shards[order_slot], ids, self.world)
        return RF.table_view(rows, self.bits) if (self.bits and not self.rows_are_views) else rows

    def add_lookup(self, x, idx, doc_start, gains, rows=None):
        ids = self.ids(idx, doc_start) if rows is None else rows
        b, t = idx.shape
        for j in range(len(self.orders)):
            flat = ids[j].reshape(-1)
            if torch.is_grad_enabled():
                r = _LookupFn.apply(self._anchor, self, j, flat)
            else:
                r = self.gather(j, flat)
            x = x + gains[j].to(x.dtype) * r.view(b, t, self.dim).to(x.dtype)
        return x

    def record_grad(self, order_slot, ids, g):
        push = getattr(self.exchange, "push_grads", None)
        if push is not None:         # peer-memory transport: the rows leave for their owners now, inside backward
            push(order_slot, ids.detach(), g.detach())
        else:
            self.pending.append((order_slot, ids.detach(), g.detach()))

    # -- update ---------------------------------------------------------------------------------------------
    @torch.no_grad()
    def step(self, lr: float):
        """Apply every recorded gradient: route ``(id, grad)`` pairs to the owners, sum duplicates, average over ranks,
        update the touched rows."""
        self.steps += 1
        apply_fused = getattr(self.exchange, "apply_updates", None)
        if apply_fused is not None:
            apply_fused(self, lr)
            return
        pend, self.pending = self.pending, []
        for j in range(len(self.orders)):
            parts = [(i, g) for (o, i, g) in pend if o == j]
            if parts:
                ids = torch.cat([p[0] for p in parts])
                grads = torch.cat([p[1] for p in parts]).float()
            else:
                ids = torch.zeros(0, dtype=torch.int64, device=self.device)
                grads = torch.zeros(0, self.dim, device=self.device)
            lids, lgrads = self.exchange.send_grads(ids, grads, self.world)      # owned entries, local row ids
            ok = torch.isfinite(lgrads).all()
            if self.world > 1:
                ok = self.exchange.all_ok(ok)
            if not bool(ok):
                self.stats["skipped"] += 1
                continue
            uniq, inv = torch.unique(lids, return_inverse=True)
            acc = torch.zeros(len(uniq), self.dim, dtype=torch.float32, device=lgrads.device)
            acc.index_add_(0, inv, lgrads)
            acc /= self.world
            if self.opt == "rowrms":
                RF.table_rowrms_update(self.shards[j], uniq, acc, self.row_sq[j], lr=lr, beta=self.betas[1], eps=self.eps,
                                       decay=self.decay)
            else:
                self._sparse_adam(j, uniq, acc, lr)
            self.stats["updates"] += 1
            self.stats["touched"] += int(len(uniq))
        done = getattr(self.exchange, "after_update", None)
        if done is not None:
            done()          # peers read these shards directly: no rank starts its next lookup before every owner is done

    def _sparse_adam(self, j, rows, g, lr):
        from .. import ops
        b1, b2 = self.betas
        if self.host_state:
            cpu_rows = rows.cpu()
            with torch.cuda.stream(self.side_stream):
                self.side_stream.wait_stream(torch.cuda.current_stream())
                m = self.exp_avg[j].index_select(0, cpu_rows).pin_memory().to(self.device, non_blocking=True)
                v = self.exp_avg_sq[j].index_select(0, cpu_rows).pin_memory().to(self.device, non_blocking=True)
                ops.sparse_adam_rows(self.shards[j], rows, g, m, v, step=self.steps, lr=lr, beta1=b1, beta2=b2,
                                     eps=self.eps, decay=self.decay)
                mh, vh = m.to("cpu", non_blocking=True), v.to("cpu", non_blocking=True)
            self.side_stream.synchronize()
            self.exp_avg[j].index_copy_(0, cpu_rows, mh)
            self.exp_avg_sq[j].index_copy_(0, cpu_rows, vh)
            torch.cuda.current_stream().wait_stream(self.side_stream)
        else:
            m = self.exp_avg[j].index_select(0, rows)
            v = self.exp_avg_sq[j].index_select(0, rows)
            ops.sparse_adam_rows(self.shards[j], rows, g, m, v, step=self.steps, lr=lr, beta1=b1, beta2=b2,
                                 eps=self.eps, decay=self.decay)
            self.exp_avg[j].index_copy_(0, rows, m)
            self.exp_avg_sq[j].index_copy_(0, rows, v)

    # -- checkpoint -----------------------------------------------------------------------------------------
    def state_for_checkpoint(self, quantize: bool = False) -> dict:
        """This rank's share.  ``quantize`` stores int8 rows with a bf16 row scale (reference: ``quantize_for_save``,
        round2/source/train.py:3752-3800)."""
        out = {}
        for j, o in enumerate(self.orders):
            t = self.shards[j].detach().cpu()
            if self.bits:
                out[f"table_{o}"], out[f"table_{o}_scale"] = RF.table_pack_view(t, self.bits)
            elif quantize:
                scale = (t.float().abs().amax(1, keepdim=True) / 127.0).clamp_min(1e-12)
                out[f"table_{o}"] = torch.round(t.float() / scale).clamp(-127, 127).to(torch.int8)
                out[f"table_{o}_scale"] = scale.to(torch.bfloat16)
            else:
                out[f"table_{o}"] = t
        return out

    def load_share(self, state: dict):
        for j, o in enumerate(self.orders):
            t = state[f"table_{o}"]
            if t.dtype == torch.uint8:
                t = RF.table_unpack_view(t, state[f"table_{o}_scale"], self.bits)
                self.rows_are_views = True
            elif t.dtype == torch.int8:
                t = t.float() * state[f"table_{o}_scale"].float()
            if t.shape[0] == self.rows and self.world > 1:
                t = t[self.rank::self.world]
            self.shards[j].copy_(t.to(self.dtype))
