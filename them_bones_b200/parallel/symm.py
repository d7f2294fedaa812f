"""Peer-memory communicator: symmetric slabs + the fused compute/collective kernels of ``csrc/comm.cu``.

Plumbing: every slab is a symmetric allocation (``torch.distributed._symmetric_memory``: same size on every rank, peer
mappings exchanged once at rendezvous); the kernels receive the W peer pointers by value.  The four communication-bound
paths of the optimizer step then run without an NCCL call:

* path 1 (gradient reduce-scatter + optimizer prologue): ``rs_muon_prep`` reads the owned chunk out of all W gradient
  slabs by NVLink peer loads, averages in fp32, applies the Muon momentum/Nesterov mix and emits the bf16
  Newton-Schulz input and its squared Frobenius norm; ``rs_adamw_publish`` does the same reduction fused with AdamW on
  the owned rows.  Both also accumulate sum(g^2) for the finiteness gate.
* path 2 (parameter publish): updated bf16 shards are stored straight into every rank's weight slab by peer stores
  (``peer_publish``; inside ``rs_adamw_publish`` for the row tables), so the next forward's GEMMs read the slab they
  always read and no all-gather buffer exists.
* ``peer_allreduce_small`` for the stacked scalars; ``peer_all_to_all`` / ``peer_gather_rows`` for the MoE slot buffer
  and the hashed tables (``PeerMoeExchange``, ``PeerTableExchange``).

Ordering between ranks is an epoch barrier kernel with bounded waits (``bones_peer_barrier``).  Reference counterparts:
the lean optimizer's collectives (round2/source/train.py:13117-13293) and its live cross-check of the overlapped
collectives against the eager ones (``_ovl_check``, :13092-13116), kept here as ``cross_check``.
"""
from __future__ import annotations

import ctypes

import torch
import torch.distributed as dist

from ..ops import _lib as L
from ..ref import functional as RF

_I, _L, _F, _D = ctypes.c_int, ctypes.c_longlong, ctypes.c_float, ctypes.c_double


def _ptr_array(ptrs):
    return (ctypes.c_void_p * len(ptrs))(*[ctypes.c_void_p(int(p)) for p in ptrs])


class PeerComm:
    fused = True

    def __init__(self, rt, group=None, wait_seconds: float = 20.0):
        import torch.distributed._symmetric_memory as symm_mem
        self.symm_mem = symm_mem
        self.rt = rt
        self.group = group or dist.group.WORLD
        self.world, self.rank = rt.world, rt.rank
        self.device = rt.device
        self.wait_seconds = wait_seconds
        self._handles = {}                    # data_ptr -> (tensor, handle, ptr array, multicast address or 0)
        from ..config import switches
        self.nvls = bool(switches()["NVLS"])  # reduce / broadcast through the switch where a buffer has a multicast mapping
        self._canaries = []
        self.epoch_dev = torch.zeros(1, dtype=torch.int32, device=self.device)    # advanced by the barrier kernel itself
        self.flags = self.alloc((64,), torch.int32, self.device)
        self.gsq = torch.zeros(1, dtype=torch.float32, device=self.device)
        self.launches = 0

    @classmethod
    def create(cls, rt):
        return cls(rt)

    # -- symmetric allocation ---------------------------------------------------------------------------------
    CANARY = 0xA5

    def alloc(self, shape, dtype, device):
        """Symmetric allocation of ``shape``, zeroed, followed by 256 bytes of canary that no kernel should ever touch:
        peers write into these buffers with offsets computed on other GPUs, and ``check_canaries()`` is how an overrun
        shows up (no memory checker runs on these machines)."""
        n = 1
        for d in shape:
            n *= int(d)
        item = torch.empty((), dtype=dtype).element_size()
        pad = 256 // item
        base = self.symm_mem.empty(n + pad, dtype=dtype, device=device)
        base.zero_()
        base[n:].view(torch.uint8).fill_(self.CANARY)
        hdl = self.symm_mem.rendezvous(base, self.group)
        t = base[:n].view(*shape)
        mc = int(getattr(hdl, "multicast_ptr", 0) or 0)
        if mc:
            mc += t.data_ptr() - int(hdl.buffer_ptrs[self.rank])
        self._handles[t.data_ptr()] = (t, hdl, _ptr_array(hdl.buffer_ptrs), mc)
        self._canaries.append((tuple(shape), dtype, base[n:].view(torch.uint8)))
        return t

    def check_canaries(self) -> None:
        """Raises if any byte after a symmetric buffer changed (synchronises)."""
        if not self._canaries:
            return
        bad = torch.stack([(c != self.CANARY).any() for _, _, c in self._canaries])
        if bool(bad.any()):
            which = [f"{shape} {dtype}" for (shape, dtype, _), b in zip(self._canaries, bad.tolist()) if b]
            raise RuntimeError(f"a kernel wrote past the end of a symmetric buffer: {which}")

    def peer_addresses(self, t):
        """The W device addresses of symmetric tensor ``t`` as Python ints (index = rank)."""
        ent = self._handles.get(t.data_ptr())
        if ent is None:
            raise RuntimeError("tensor is not a symmetric allocation of this communicator")
        return [int(p) for p in ent[1].buffer_ptrs]

    def multicast_mapped(self) -> int:
        """How many symmetric allocations have a multicast mapping that the kernels use (0 with ``BONES_NVLS=0``)."""
        return sum(1 for e in self._handles.values() if len(e) > 3 and e[3]) if self.nvls else 0

    def multicast(self, t):
        """The multicast address of symmetric tensor ``t`` as a ctypes pointer: a load from it (``multimem.ld_reduce``)
        sums all ranks' copies inside the switch, a store to it (``multimem.st``) lands in every copy.  Null when the
        allocation has no multicast mapping or ``BONES_NVLS=0``; the kernels then loop over the peer pointers."""
        ent = self._handles.get(t.data_ptr())
        mc = ent[3] if (ent is not None and self.nvls and len(ent) > 3) else 0
        return ctypes.c_void_p(mc or None)

    def peers(self, t):
        """ctypes array of the W peer pointers of symmetric tensor ``t`` (or of the allocation a view starts in)."""
        ent = self._handles.get(t.data_ptr())
        if ent is None:
            raise RuntimeError("tensor is not a symmetric allocation of this communicator")
        return ent[2]

    # -- ordering -----------------------------------------------------------------------------------------------
    def barrier(self):
        L.call("bones_peer_barrier", self.peers(self.flags), _I(self.rank), _I(self.world), L.ptr(self.epoch_dev),
               _D(self.wait_seconds), L.stream())
        self.launches += 1

    def pre_step(self):
        """Every rank's gradient slabs are complete and visible before any peer reads them."""
        self.gsq.zero_()
        self.barrier()

    def post_step(self):
        """Every peer's stores into my weight slabs have landed before the next forward reads them."""
        self.barrier()

    # -- collectives used by the lean optimizer ---------------------------------------------------------------
    def all_reduce_mean(self, t):
        """Small stacked scalars: ``t`` must be symmetric; every rank computes the same sum."""
        if t.numel() == 0:
            return t
        ent = self._handles.get(t.data_ptr())
        if ent is None:
            dist.all_reduce(t, group=self.group)
            return t.div_(self.world)
        out = torch.empty_like(t)
        L.call("bones_peer_allreduce_small", ent[2], L.ptr(out), _I(t.numel()), _I(self.world), _F(1.0 / self.world),
               L.stream())
        self.launches += 1
        return out

    def all_reduce_min(self, t):
        dist.all_reduce(t, op=dist.ReduceOp.MIN, group=self.group)
        return t

    def fused_row_adamw(self, u, step):
        g = u.group
        n = u.master.numel()
        off = self.rank * n
        b1, b2 = g["betas"]
        L.call("bones_rs_adamw_publish_mc", self.peers(u.G), self.peers(u.W), _L(off), _L(n), _I(self.world),
               _F(1.0 / self.world), L.ptr(u.master), L.ptr(u.exp_avg), L.ptr(u.exp_avg_sq), _F(g["lr"]), _F(b1), _F(b2),
               _F(g["eps"]), _F(g["weight_decay"]), _I(step), L.ptr(self.gsq), self.multicast(u.G), self.multicast(u.W),
               L.stream())
        self.launches += 1

    def fused_muon(self, u, step, ns_dtype, own_only=False):
        # own_only: the owner's slab already holds the sum over ranks (pushed by the weight-gradient GEMMs), so only
        # this rank's slab is read (still divided by the world size)
        from ..ops import muon_native as MN
        g = u.group
        mat = u.r * u.c
        kr = getattr(u, "kr", u.k)                         # matrices this rank owns; the rest of its slots is padding
        if kr == 0:
            return
        n = kr * mat
        off = self.rank * u.k * mat
        if not hasattr(u, "X"):
            u.X = torch.empty(u.k, u.r, u.c, dtype=torch.bfloat16, device=u.W.device)
            u.sumsq = torch.zeros(u.k, dtype=torch.float32, device=u.W.device)
        u.sumsq.zero_()
        if own_only:
            if not hasattr(u, "own_ptr"):
                u.own_ptr = _ptr_array([self.peer_addresses(u.G)[self.rank]])
            src, nsrc, mc_g = u.own_ptr, 1, ctypes.c_void_p(None)
        else:
            src, nsrc, mc_g = self.peers(u.G), self.world, self.multicast(u.G)
        L.call("bones_rs_muon_prep_mc", src, _L(off), _L(n), _I(nsrc), _F(1.0 / self.world),
               _F(g["momentum"]), L.ptr(u.momentum), L.ptr(u.X), L.ptr(u.sumsq), _L(mat), L.ptr(self.gsq), mc_g, L.stream())
        L.call("bones_muon_normalize", L.ptr(u.X), L.ptr(u.sumsq), _L(n), _L(mat), L.stream())
        x = MN.newton_schulz(u.X[:kr], g["ns_steps"])
        MN.muon_finish(x, u.master[:kr], u.second[:kr], beta2=g["beta2"], lr=g["lr"], wd=g["weight_decay"])
        L.call("bones_peer_publish_mc", L.ptr(u.master), self.peers(u.W), _L(off), _L(n), _I(self.world), self.multicast(u.W),
               L.stream())
        self.launches += 3

    # -- cross-check against the library collectives on the same live inputs ----------------------------------
    @torch.no_grad()
    def cross_check(self, opt) -> int:
        bad = 0
        for u in opt.muon_units + opt.row_units:
            full = torch.empty_like(u.W)
            own = u.W.view(self.world, -1)[self.rank].contiguous()
            dist.all_gather_into_tensor(full.view(-1), own, group=self.group)
            bad += int((full != u.W).sum())
        t = torch.tensor([bad], device=self.device)
        dist.all_reduce(t, group=self.group)
        return int(t.item())

    # -- MoE / tables ---------------------------------------------------------------------------------------------
    def install_moe(self, model):
        from . import moe_a2a
        moe_a2a.install_fused(PeerMoeExchange(self))

    def table_exchange(self, tables, entries_per_step: int = 0):
        return PeerTableExchange(self, tables, entries_per_step)


def create_or_fallback(rt, factory=None):
    """Start-up probe of the peer-memory substrate: build the communicator, run one fused all-reduce and one epoch
    barrier on known values, and let the ranks agree on the outcome.  Any rank's failure (no symmetric-memory support,
    no peer access, a wrong sum, an expired wait) sends *every* rank to the library-collective path: returns ``None`` and
    rank 0 prints one line (reference: ``configure_sharding`` probes its collectives on tiny tensors at start-up and
    falls back, round1/source/train.py:9742-9774).  ``factory`` builds the communicator (tests inject a failing one)."""
    def agree(flag: bool) -> bool:
        ok = torch.tensor([1 if flag else 0], dtype=torch.int32)
        if rt.ddp and rt.world > 1:
            group = getattr(rt, "control_group", None)
            if group is None:
                ok = ok.to(rt.device)
            dist.all_reduce(ok, op=dist.ReduceOp.MIN, group=group)
        return int(ok[0]) == 1

    def give_up(why: str):
        if rt.rank == 0:
            print(f"peer-memory communicator unavailable ({why or 'another rank failed its probe'}); "
                  "using the library collectives", flush=True)
        return None

    # stage 1, local and cheap: what a rank can tell without talking to the others (a rank that failed alone in stage 2
    # would leave the others waiting in the rendezvous, so obvious causes are caught here, where all ranks still agree)
    why = ""
    try:
        import torch.distributed._symmetric_memory  # noqa: F401
        if factory is None and rt.device_type == "cuda":
            me = torch.cuda.current_device()
            n_dev = torch.cuda.device_count()
            if rt.world > n_dev:
                why = f"{rt.world} ranks on {n_dev} visible GPUs"
            elif not all(torch.cuda.can_device_access_peer(me, d) for d in range(n_dev) if d != me and d < rt.world):
                why = "no peer access between the GPUs"
    except Exception as exc:  # noqa: BLE001
        why = f"{type(exc).__name__}: {exc}"
    if not agree(not why):
        return give_up(why)
    comm = None
    try:
        comm = (factory or PeerComm.create)(rt)
        probe = comm.alloc((256,), torch.float32, rt.device)
        probe.fill_(float(rt.rank + 1))
        comm.barrier()
        got = comm.all_reduce_mean(probe)
        comm.barrier()
        torch.cuda.synchronize(rt.device)
        L.check_error_word()
        want = (rt.world + 1) / 2.0
        if not bool(((got - want).abs() < 1e-5).all()):
            why = f"fused all-reduce returned {float(got[0])}, expected {want}"
    except Exception as exc:  # noqa: BLE001 - any failure of the substrate means: use the library collectives
        why = f"{type(exc).__name__}: {exc}"
    if not agree(not why):
        return give_up(why)
    # stage 3: the switch-multicast forms of the reduction and the publish on known values; a wrong result on any rank
    # switches them off on every rank (the peer-loop forms stay)
    if getattr(comm, "nvls", False) and comm.world > 1:
        bad = ""
        try:
            n = 1024
            g = comm.alloc((n,), torch.float32, rt.device)
            w = comm.alloc((comm.world * n,), torch.bfloat16, rt.device)
            if comm.multicast(g).value and comm.multicast(w).value:
                g.fill_(float(rt.rank + 1))
                mom, x = torch.zeros(n, device=rt.device), torch.empty(n, dtype=torch.bfloat16, device=rt.device)
                sumsq, gsq = torch.zeros(1, device=rt.device), torch.zeros(1, device=rt.device)
                comm.barrier()
                L.call("bones_rs_muon_prep_mc", comm.peers(g), _L(0), _L(n), _I(comm.world), _F(1.0 / comm.world), _F(0.0),
                       L.ptr(mom), L.ptr(x), L.ptr(sumsq), _L(n), L.ptr(gsq), comm.multicast(g), L.stream())
                src = torch.full((n,), float(rt.rank + 1), device=rt.device)
                L.call("bones_peer_publish_mc", L.ptr(src), comm.peers(w), _L(rt.rank * n), _L(n), _I(comm.world),
                       comm.multicast(w), L.stream())
                comm.barrier()
                torch.cuda.synchronize(rt.device)
                L.check_error_word()
                mean = (comm.world + 1) / 2.0
                want_w = torch.arange(1, comm.world + 1, device=rt.device, dtype=torch.float32).repeat_interleave(n)
                if not bool(((x.float() - mean).abs() < 1e-2).all()):
                    bad = f"multicast reduction returned {float(x[0])}, expected {mean}"
                elif not bool((w.float() == want_w).all()):
                    bad = "a multicast store did not reach every rank's copy"
            else:
                bad = "no multicast mapping"
        except Exception as exc:  # noqa: BLE001
            bad = f"{type(exc).__name__}: {exc}"
        if not agree(not bad):
            comm.nvls = False
            if rt.rank == 0:
                print(f"switch multicast not used ({bad or 'another rank failed its probe'}); reductions and publishes "
                      "loop over the peers", flush=True)
    return comm


class SoloComm(PeerComm):
    """The same fused optimizer kernels on one GPU: the "peer" list is this GPU alone, slabs are ordinary device
    tensors and the epoch barrier is a no-op.  The reduction kernels then read one gradient slab, apply the Muon
    prologue / AdamW and write the bf16 replicas in a single pass each, instead of the dozen element-wise passes of the
    PyTorch statement of the same update."""

    def __init__(self, rt):
        self.symm_mem, self.rt, self.group = None, rt, None
        self.world, self.rank, self.device = 1, 0, rt.device
        self._handles = {}
        self._canaries = []
        self.nvls = False
        self.gsq = torch.zeros(1, dtype=torch.float32, device=self.device)
        self.launches = 0

    def alloc(self, shape, dtype, device):
        n = 1
        for d in shape:
            n *= int(d)
        pad = 256 // torch.empty((), dtype=dtype).element_size()
        base = torch.zeros(n + pad, dtype=dtype, device=device)
        base[n:].view(torch.uint8).fill_(self.CANARY)
        t = base[:n].view(*shape)
        self._handles[t.data_ptr()] = (t, None, _ptr_array([t.data_ptr()]))
        self._canaries.append((tuple(shape), dtype, base[n:].view(torch.uint8)))
        return t

    def peer_addresses(self, t):
        if t.data_ptr() not in self._handles:
            raise RuntimeError("tensor is not an allocation of this communicator")
        return [t.data_ptr()]

    def barrier(self):
        pass

    def all_reduce_mean(self, t):
        return t

    def all_reduce_min(self, t):
        return t

    def cross_check(self, opt) -> int:
        return 0

    def install_moe(self, model):
        pass

    def peers(self, t):
        ent = self._handles.get(t.data_ptr())
        if ent is None:
            raise RuntimeError("tensor is not an allocation of this communicator")
        return ent[2]


class PeerMoeExchange:
    """Expert-parallel exchange by peer stores, written straight in the layout the consumer reads.

    Buffers are symmetric allocations that persist: the dispatch buffer and the return buffer of a layer are per layer
    (``key``), because the expert GEMMs and the combine keep them for their backward passes and nothing is copied out;
    the two gradient exchanges share one buffer each across layers.  One epoch barrier per exchange, after the stores
    ("every peer's rows have landed"); none is needed before them: a peer can only reach the next writer of a buffer after
    a barrier that this rank arrives at later in its stream than the last reader of that buffer (the next writer of a
    per-layer buffer is the same layer one micro-step on, behind that layer's backward exchanges; the next writer of a
    shared gradient buffer is the layer below, behind the other gradient exchange of this layer)."""

    def __init__(self, comm: PeerComm):
        self.comm = comm
        self.bufs = {}

    def _recv(self, numel, dtype, key):
        k = (numel, dtype, key)
        if k not in self.bufs:
            self.bufs[k] = self.comm.alloc((numel,), dtype, self.comm.device)
        return self.bufs[k]

    def _a2a(self, x, key):
        """Plain equal-split all-to-all (chunk d of ``x`` to slot ``rank`` of peer d); used by the self-test."""
        comm = self.comm
        x = x.contiguous()
        recv = self._recv(x.numel(), x.dtype, key)
        comm.barrier()                                   # the receive buffer's previous contents have been consumed
        L.call("bones_peer_all_to_all", L.ptr(x), comm.peers(recv), _L(x.numel() * x.element_size() // comm.world),
               _I(comm.rank), _I(comm.world), L.stream())
        comm.barrier()                                   # every peer's rows have landed
        return recv.view(x.shape).clone()

    def _blocks(self, x, world, m, mode, key):
        """``x [m * W * rows, d]`` bf16 -> the other layout on the peers (see ``peer_blocks_kernel``); returns this rank's
        receive buffer as a ``[m * W * rows, d]`` view."""
        comm = self.comm
        x = x.contiguous()
        d = x.shape[-1]
        rows = x.shape[0] // (m * world)
        recv = self._recv(x.numel(), x.dtype, key)
        L.call("bones_peer_blocks", L.ptr(x), comm.peers(recv), _L(rows), _I(m), _I(d), _I(comm.rank), _I(world), _I(mode), L.stream())
        comm.barrier()
        comm.launches += 1
        return recv.view(x.shape)

    def exchange(self, xs, world, m, forward, key=None):
        return _PeerBlocksFn.apply(xs, self, world, m, forward, key)

    def dispatch(self, h, tok, world, m, slot=None, key=None):
        """Permute + exchange in one kernel: token rows go straight into the owning rank's expert buffer."""
        return _PeerDispatch.apply(h, tok, slot, self, world, m, key)


class _PeerDispatch(torch.autograd.Function):
    @staticmethod
    def forward(ctx, h, tok, slot, ex, world, m, key):
        comm = ex.comm
        h = h.contiguous()
        n_slots, d = tok.numel(), h.shape[1]
        rows = n_slots // (world * m)                                      # rows per (expert, source rank) block
        recv = ex._recv(n_slots * d, h.dtype, ("disp", key))
        L.call("bones_peer_dispatch_grouped", L.ptr(h), L.ptr(tok), comm.peers(recv), _L(rows), _I(m), _L(n_slots), _L(h.shape[0]),
               _I(d), _I(comm.rank), _I(world), L.stream())
        comm.barrier()
        comm.launches += 1
        ctx.save_for_backward(tok, slot if slot is not None else tok)
        ctx.ex, ctx.world, ctx.m, ctx.n, ctx.has_slot = ex, world, m, h.shape[0], slot is not None
        return recv.view(n_slots, d)                                        # [m, W(src), rows, d]: grouped by local expert

    @staticmethod
    def backward(ctx, g):
        tok, slot = ctx.saved_tensors
        ex, world, m, d = ctx.ex, ctx.world, ctx.m, g.shape[-1]
        dxs = ex._blocks(g.reshape(-1, d), world, m, 1, "gdisp")            # gradients of my slots, [E * rows, d]
        if ctx.has_slot:            # every token sums its (at most k) slots: the combine kernel with unit gates
            from ..ops import cuda as C
            ones = torch.ones(slot.shape, dtype=torch.float32, device=g.device)
            dh = torch.empty(ctx.n, d, dtype=g.dtype, device=g.device)
            L.call("bones_moe_combine", L.ptr(dxs), L.ptr(slot), L.ptr(ones), L.ptr(dh), _I(ctx.n), _I(d), _I(slot.shape[1]),
                   _L(dxs.shape[0]), L.stream())
            return dh, None, None, None, None, None, None
        dh = torch.zeros(ctx.n + 1, d, dtype=torch.float32, device=g.device)
        dh.index_add_(0, tok, dxs.float())
        return dh[:ctx.n].to(g.dtype), None, None, None, None, None, None


class _PeerBlocksFn(torch.autograd.Function):
    """forward=True: slot layout ``[W(dst), m, rows]`` to the experts' ``[m, W(src), rows]``; forward=False: the experts'
    layout back to the sources' slot layout.  The backward of each is the other, through a buffer shared by all layers."""

    @staticmethod
    def forward(ctx, xs, ex, world, m, forward, key):
        ctx.ex, ctx.world, ctx.m, ctx.fwd = ex, world, m, forward
        return ex._blocks(xs, world, m, 0 if forward else 1, ("f" if forward else "r", key))

    @staticmethod
    def backward(ctx, g):
        ex, world, m = ctx.ex, ctx.world, ctx.m
        out = ex._blocks(g.reshape(-1, g.shape[-1]), world, m, 1 if ctx.fwd else 0, "gf" if ctx.fwd else "gr")
        return out, None, None, None, None, None


class PeerTableExchange:
    """Tables over peer memory, both directions.  Lookups read the owners' shards directly through peer pointers (one
    gather kernel, no id exchange).  Gradients: every ``(row id, gradient row)`` recorded by backward is pushed straight
    into the owning rank's staging buffer (a system-scope atomic reserves the slot, peer stores fill it); at the step
    boundary the owner sorts the staged ids on the device and one kernel sums each row's duplicates and updates the table
    in place (``csrc/tables.cu``).  No library collective and no host synchronisation in a step.  With one rank the
    same kernels run on a one-entry peer list."""

    fused_grads = True

    def __init__(self, comm: PeerComm, tables, entries_per_step: int = 0, headroom: float = 1.5):
        from .table_a2a import CollectiveExchange
        self.comm = comm
        self.world = comm.world
        self.fallback = (CollectiveExchange(comm.group, comm.world, comm.rank, comm.device) if comm.world > 1 else None)
        # re-home the shards in symmetric memory so peers can read them
        for j, sh in enumerate(tables.shards):
            sym = comm.alloc(tuple(sh.shape), sh.dtype, sh.device)
            sym.copy_(sh)
            tables.shards[j] = sym
        dim = tables.dim
        self.rows_per_shard = tables.local_rows
        self.native = (tables.dtype == torch.bfloat16 and dim % 256 == 0 and dim <= 2048 and entries_per_step > 0
                       and not tables.host_state)
        if not self.native:
            self.push_grads = None          # gradients travel by the library all-to-all; the update is the PyTorch one
            self.apply_updates = None
            return
        # staging per table: an owner receives about its share of all ranks' entries, i.e. one rank's worth; hashing
        # spreads the rows evenly, the headroom covers the heavy hitters that all land on one owner
        self.cap = int(entries_per_step * headroom) + 4096
        self.stage_ids, self.stage_g, self.stage_cnt, self.stats = [], [], [], []
        for _ in tables.orders:
            ids = comm.alloc((self.cap,), torch.int64, comm.device)
            ids.fill_(0x7FFFFFFFFFFFFFFF)
            self.stage_ids.append(ids)
            self.stage_g.append(comm.alloc((self.cap, dim), torch.bfloat16, comm.device))
            self.stage_cnt.append(comm.alloc((4,), torch.int32, comm.device))
            self.stats.append(torch.zeros(2, dtype=torch.int32, device=comm.device))
        self.overflow = torch.zeros(1, dtype=torch.int32, device=comm.device)
        comm.barrier()

    def lookup(self, shard, ids, world):
        out = torch.empty(ids.numel(), shard.shape[1], dtype=shard.dtype, device=shard.device)
        L.call("bones_peer_gather_rows", self.comm.peers(shard), L.ptr(ids.contiguous()), L.ptr(out), _I(ids.numel()),
               _I(shard.shape[1]), _I(world), _L(shard.shape[0]), L.stream())
        return out

    # -- gradients: native route -------------------------------------------------------------------------------
    def push_grads(self, j, ids, g):
        g = g.contiguous()
        if g.dtype != torch.bfloat16:
            g = g.to(torch.bfloat16)
        comm = self.comm
        L.call("bones_table_push", L.ptr(ids.contiguous()), L.ptr(g), _L(ids.numel()), _I(g.shape[1]), comm.peers(self.stage_ids[j]),
               comm.peers(self.stage_g[j]), comm.peers(self.stage_cnt[j]), _I(self.cap), _I(self.world), L.ptr(self.overflow),
               _L(self.rows_per_shard), L.stream())

    def apply_updates(self, tables, lr):
        comm = self.comm
        comm.barrier()                       # every rank's pushes of this step have landed in my staging buffers
        mode = 0 if tables.opt == "rowrms" else 1
        b1, b2 = tables.betas
        for j in range(len(tables.orders)):
            sorted_ids, order = torch.sort(self.stage_ids[j])          # device-side; empty slots hold the largest key
            s0 = tables.row_sq[j] if mode == 0 else tables.exp_avg[j]
            s1 = None if mode == 0 else tables.exp_avg_sq[j]
            L.call("bones_table_update", L.ptr(sorted_ids), L.ptr(order), L.ptr(self.stage_g[j]), L.ptr(self.stage_cnt[j]), _I(self.cap),
                   L.ptr(tables.shards[j]), L.ptr(s0), L.ptr(s1), _I(mode), _I(tables.dim), _F(lr), _F(b1), _F(b2), _F(tables.eps),
                   _F(tables.decay), _I(tables.steps), _F(1.0 / self.world), ctypes.c_uint((tables.steps * 2654435761 + j) & 0xFFFFFFFF),
                   L.ptr(self.stats[j]), _L(self.rows_per_shard), L.stream())
            L.call("bones_table_reset", L.ptr(self.stage_ids[j]), L.ptr(self.stage_cnt[j]), _I(self.cap), L.stream())
        comm.barrier()                       # updates and resets are done before any rank looks up or pushes again

    def read_stats(self) -> dict:
        """Rows updated / skipped so far and entries dropped for a full staging buffer (synchronises)."""
        st = torch.stack(self.stats).sum(0).tolist() if self.native else [0, 0]
        return dict(touched=int(st[0]), skipped=int(st[1]), overflow=int(self.overflow.item()) if self.native else 0)

    # -- gradients: library route (tables the native kernels do not cover) -------------------------------------
    def send_grads(self, ids, grads, world):
        if self.fallback is None:
            return ids, grads
        return self.fallback.send_grads(ids, grads, world)

    def all_ok(self, ok):
        return ok if self.fallback is None else self.fallback.all_ok(ok)

    def after_update(self):
        """Library route only.  Lookups are peer loads with no collective of their own, so without this a fast rank
        could gather rows from a shard its owner is still updating (stale or torn rows); the epoch barrier (bounded
        wait) orders every owner's update before any rank's next gather."""
        self.comm.barrier()
