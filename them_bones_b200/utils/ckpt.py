"""Checkpoint save / load in the reference layout.

``torch.save({"model_state": {name: cpu tensor}, "model_config": {non-default GPTConfig fields}, "meta": {...}})``
(reference: ``save_checkpoint`` round2/source/train.py:20734-20746, ``save_rescue_checkpoint`` :20749, ``load_for_eval``
:21031-21126).  Experts are gathered to rank 0 one tensor at a time (``moe_gather_experts`` :20027-20046) and stored as
``transformer.h.{i}.mlp.w_fc [E,H,d]`` / ``w_proj [E,d,H]``; table shares are stored as extra state keys.  Files are
written to ``<path>.tmp`` and renamed so a reader never sees a partial file.  Optimizer state is saved only on request
(``BONES_SAVE_OPT_STATE=1``: one ``<path>.opt.rank<r>`` file per rank with the owner state of that rank, read back by
``train.py --resume``; the reference never saves it).
"""
from __future__ import annotations

import os

import torch
import torch.distributed as dist

from ..config import GPTConfig, model_config_dict


def _is_dist():
    return dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1


def gather_experts(model, group=None) -> dict:
    """Full ``[E, ...]`` expert tensors on every rank (cold path: library all-gather)."""
    from ..models.moe import MoeMLP
    out = {}
    for i, blk in enumerate(model.transformer.h):
        if not isinstance(blk.mlp, MoeMLP):
            continue
        for name in ("w_fc", "w_proj"):
            local = getattr(blk.mlp, name).detach()
            if blk.mlp.ep_world > 1:
                full = torch.empty(blk.mlp.n_exp, *local.shape[1:], dtype=local.dtype, device=local.device)
                dist.all_gather_into_tensor(full, local.contiguous(), group=blk.mlp.ep_group)
            else:
                full = local
            out[f"transformer.h.{i}.mlp.{name}"] = full.cpu()
    return out


def model_state(model, optimizer=None, group=None) -> dict:
    """Name -> CPU tensor.  With a lean optimizer the fp32 masters are what is saved (reference:
    ``consolidated_state_dict``)."""
    masters = optimizer.consolidated_state_dict() if hasattr(optimizer, "consolidated_state_dict") else {}
    state = {}
    experts = gather_experts(model, group)
    for name, p in model.named_parameters():
        if name in experts:
            state[name] = experts[name]
        elif p in masters:
            state[name] = masters[p].detach().cpu().clone()
        else:
            state[name] = p.detach().cpu().clone()
    return state


def _gather_rows(table) -> dict:
    """A row-sharded table's checkpoint entries with every rank's share interleaved back (owner = row % world)."""
    share = table.state_for_checkpoint()
    if not _is_dist() or getattr(table, "world", 1) == 1:       # an unsharded table already holds every row
        return share
    parts = [None] * dist.get_world_size()
    dist.all_gather_object(parts, share)
    out = {}
    for k in share:
        full = torch.empty(table.rows, *share[k].shape[1:], dtype=share[k].dtype)
        for r, part in enumerate(parts):
            full[r::len(parts)] = part[k]
        out[k] = full
    return out


def load_model_state(model, state: dict, ep_world: int = 1, ep_rank: int = 0) -> None:
    """Checkpoint ``model_state`` -> a freshly built model (resume).  Expert tensors are stored gathered ``[E, ...]``;
    an expert-parallel rank keeps its own ``E / ep_world`` of them.  Table and output-table shares are not parameters
    and are loaded by their owners."""
    own = dict(model.named_parameters())
    with torch.no_grad():
        for name, p in own.items():
            t = state[name]
            if t.shape != p.shape and t.dim() == p.dim() and t.shape[1:] == p.shape[1:] and t.shape[0] == p.shape[0] * ep_world:
                t = t[ep_rank * p.shape[0]:(ep_rank + 1) * p.shape[0]]
            p.copy_(t.to(p.dtype))


def opt_state_path(path: str, rank: int) -> str:
    return f"{path}.opt.rank{rank}"


def save_optimizer_state(path: str, optimizer, rank: int) -> str | None:
    """Every rank writes its own owner state beside the checkpoint (``BONES_SAVE_OPT_STATE=1``)."""
    if not hasattr(optimizer, "unit_state_dict"):
        return None
    out = opt_state_path(path, rank)
    write_payload(out, optimizer.unit_state_dict())
    return out


def build_payload(model, meta: dict, optimizer=None, tables=None, state: dict | None = None) -> dict:
    """The checkpoint as host tensors.  Collective when the model is sharded: every rank must call it."""
    state = state if state is not None else model_state(model, optimizer)
    extra = {}
    if tables is not None:
        extra.update(_gather_rows(tables))
    if getattr(model, "os1", None) is not None:
        extra.update(_gather_rows(model.os1))
    return {"model_state": {**state, **extra}, "model_config": model_config_dict(model.config), "meta": meta}


def write_payload(path: str, payload: dict) -> None:
    """Atomic write: a temporary file beside ``path``, then a rename."""
    tmp = path + ".tmp"
    os.makedirs(os.path.dirname(os.path.abspath(path)), exist_ok=True)
    torch.save(payload, tmp)
    os.replace(tmp, path)


def save_checkpoint(path: str, model, meta: dict, optimizer=None, tables=None, rank: int = 0, state: dict | None = None):
    """Collective when the model is sharded: every rank must call it; only rank 0 writes."""
    payload = build_payload(model, meta, optimizer, tables, state)
    if rank == 0:
        write_payload(path, payload)


class BackgroundSave:
    """Checkpoint writes off the training thread: the host copy of the state is taken by the caller (a collective on
    sharded models), serialisation and the file write run on a worker thread while training goes on.  One write is in
    flight at a time; a new one waits for the previous (reference: the overlapped background saves ``SaveovBg``,
    round2/source/train.py:20203-20430)."""

    def __init__(self):
        self.thread, self.error, self.done, self.seconds = None, None, 0, 0.0

    def submit(self, path: str, payload: dict) -> None:
        import threading
        import time
        self.wait()

        def work():
            t0 = time.time()
            try:
                write_payload(path, payload)
                self.done += 1
            except Exception as exc:  # noqa: BLE001  (reported by wait(); training is not interrupted by a failed write)
                self.error = exc
            self.seconds += time.time() - t0

        self.thread = threading.Thread(target=work, daemon=True)
        self.thread.start()

    def wait(self) -> None:
        if self.thread is not None:
            self.thread.join()
            self.thread = None
        if self.error is not None:
            err, self.error = self.error, None
            raise RuntimeError(f"background checkpoint write failed: {err}")


def check_declared_length(model, trained_seq_len: int) -> None:
    """The scorer takes ``model_config.sequence_len`` as its maximum length, so a checkpoint must declare the window
    length it was trained on (reference: ``check_declared_length``, round2/source/train.py:20767-20774)."""
    declared = model.config.sequence_len
    if declared != trained_seq_len:
        raise RuntimeError(f"model_config.sequence_len={declared} differs from the trained window length {trained_seq_len}")


def load_for_eval(path: str, device="cpu", dtype=None, rt=None):
    """Rebuild the model from a checkpoint with no environment: ``GPTConfig(**model_config)``, strict load of the
    dense state, experts and tables attached separately, eval mode.

    Without ``rt`` every rank is an independent full replica (all experts local, whole tables), as in the reference
    (round2/source/train.py:21031-21126).  With a multi-rank ``rt`` (``runtime.init_runtime``) the model is served
    sharded: each rank keeps ``E / world`` experts and ``rows / world`` rows of every table, the ranks score / decode in
    lockstep, experts are reached by the fused peer-memory dispatch and table rows by peer gathers -- the layout a model
    whose tables do not fit one GPU needs."""
    from ..models.gpt import GPT
    from ..models.tables import HashedTables
    ckpt = torch.load(path, map_location="cpu", weights_only=True, mmap=True)
    config = GPTConfig(**ckpt["model_config"])
    state = dict(ckpt["model_state"])
    device = torch.device(device)
    sharded = rt is not None and rt.world > 1 and (bool(config.moe_layers) or bool(config.table_orders))
    world, rank = (rt.world, rt.rank) if sharded else (1, 0)
    model = GPT(config, ep_group=dist.group.WORLD if (sharded and config.moe_layers) else None,
                ep_world=world if config.moe_layers else 1, ep_rank=rank if config.moe_layers else 0)
    table_state = {k: state.pop(k) for k in list(state) if k.startswith("table_") and not k.startswith("table_lambda")}
    os1_state = {k: state.pop(k) for k in list(state) if k in ("os1_table", "os1_scale")}
    if sharded:
        load_model_state(model, state, ep_world=world if config.moe_layers else 1, ep_rank=rank)
    else:
        model.load_state_dict(state, strict=True)
    dtype = dtype or (torch.bfloat16 if device.type == "cuda" else torch.float32)
    model = model.to(device)
    model.cast_compute(dtype)
    comm = None
    if sharded and device.type == "cuda":
        from ..parallel import symm
        comm = symm.create_or_fallback(rt)
    if config.table_orders:
        tables = HashedTables(config.table_orders, config.table_rows, config.n_embd, seed=config.table_seed, bits=config.table_bits,
                              device=device, dtype=dtype, group=dist.group.WORLD if sharded else None, world=world, rank=rank,
                              opt="rowrms")
        tables.load_share(table_state)
        if comm is not None:
            tables.exchange = comm.table_exchange(tables)
        model.attach_tables(tables)
    if comm is not None and config.moe_layers:
        comm.install_moe(model)
    model.comm = comm
    if config.os1_rows:
        from ..models.os1 import OutputTable
        os1 = OutputTable(config, device=device, dtype=dtype)
        os1.load_share(os1_state)
        model.attach_os1(os1)
    model.eval()
    return model, ckpt.get("meta", {})


class RescueCopy:
    """Host copy of the weights refreshed every ``every`` steps once ``progress >= start`` and written out when the loss
    goes bad (reference: round2/source/train.py:22535-22558, 23060-23078)."""

    def __init__(self, start: float, every: int):
        self.start, self.every = start, every
        self.state, self.step = None, -1

    def maybe_refresh(self, step: int, progress: float, model, optimizer=None):
        if progress >= self.start and (self.state is None or step - self.step >= self.every):
            self.state, self.step = model_state(model, optimizer), step
            return True
        return False
