"""Expert-parallel exchange of the MoE slot buffer.

The slot buffer is laid out ``[E, b, C, d]``; expert ``e`` lives on rank ``e // m`` (``m = E / W`` experts per rank), so
the buffer splits into ``W`` equal contiguous chunks and the exchange is an equal-split all-to-all (reference:
``moe_all_to_all``, round2/source/train.py:10691-10695, whose autograd is the reversed exchange, :2958).

After the forward exchange a rank holds ``[W(src), m, b, C, d]``; it is permuted to ``[m, W*b*C, d]`` so each local
expert sees one contiguous group of rows.  The return exchange undoes both steps.

Transports: ``all_to_all_single`` (NCCL / gloo; baseline and oracle) and, when a peer-memory workspace has been
installed by ``parallel.symm``, the fused path whose dispatch kernel stores rows directly into the destination rank's
expert buffer over NVLink.
"""
from __future__ import annotations

import torch
import torch.distributed as dist

_FUSED = None        # set by parallel.symm.install_moe_workspace


def install_fused(impl):
    global _FUSED
    _FUSED = impl


class _AllToAll(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        out = torch.empty_like(x)
        dist.all_to_all_single(out, x.contiguous(), group=group)
        return out

    @staticmethod
    def backward(ctx, g):
        out = torch.empty_like(g)
        dist.all_to_all_single(out, g.contiguous(), group=ctx.group)
        return out, None


def exchange(xs: torch.Tensor, group, world: int, n_exp: int, forward: bool, key=None) -> torch.Tensor:
    """``key`` names the calling layer: the peer-memory transport keeps one receive buffer per layer and direction."""
    if world == 1:
        return xs
    d = xs.shape[-1]
    m = n_exp // world
    if _FUSED is not None and xs.is_cuda:
        return _FUSED.exchange(xs, world, m, forward, key)
    if forward:
        ys = _AllToAll.apply(xs, group)                                   # [W(src), m, bC, d]
        return ys.view(world, m, -1, d).transpose(0, 1).reshape(-1, d)    # [m, W*bC, d]
    back = xs.view(m, world, -1, d).transpose(0, 1).reshape(-1, d)        # [W(dst), m, bC, d]
    return _AllToAll.apply(back, group)


def dispatch_exchange(h: torch.Tensor, tok: torch.Tensor, group, world: int, n_exp: int, slot=None, key=None) -> torch.Tensor:
    """Slot gather + forward exchange.  With the fused transport installed this is one kernel (rows are stored straight
    into the destination rank's expert buffer, already grouped by local expert); otherwise gather then all-to-all."""
    from .. import ops
    if world > 1 and _FUSED is not None and h.is_cuda and hasattr(_FUSED, "dispatch"):
        return _FUSED.dispatch(h, tok, world, n_exp // world, slot, key)
    return exchange(ops.moe_dispatch(h, tok, slot), group, world, n_exp, True, key)
