"""Learning-rate, momentum and batch schedules.

Reference: ``lr_multiplier`` / ``lr_multiplier_by_clock`` (round2/source/train.py:21131-21157): step warm-up, flat, linear
warm-down to ``final`` over the last ``warmdown`` fraction of the horizon, where the horizon is measured in steps or in
wall-clock fraction; separate (warmdown, final) pairs for dense groups and for table rows (``env:35-37``);
``muon_momentum_schedule`` (:21160): 0.85 -> 0.97 over the first 300 steps, then -> 0.90 over the warm-down; round 1's
half batch for the first 30 % (round1/source/train.py:10148).
"""
from __future__ import annotations


def lr_multiplier(progress: float, step: int, warmup_steps: int, warmdown_frac: float, final_frac: float) -> float:
    """``progress`` in [0, 1] is the fraction of the horizon that has passed (steps or clock)."""
    if step < warmup_steps:
        return (step + 1) / warmup_steps
    start = 1.0 - warmdown_frac
    if progress <= start or warmdown_frac <= 0:
        return 1.0
    t = min(1.0, (progress - start) / warmdown_frac)
    return 1.0 - t * (1.0 - final_frac)


def muon_momentum(step: int, progress: float, warmdown_frac: float, lo=0.85, hi=0.97, end=0.90, ramp_steps=300) -> float:
    m = lo + (hi - lo) * min(1.0, step / ramp_steps)
    start = 1.0 - warmdown_frac
    if progress > start and warmdown_frac > 0:
        t = min(1.0, (progress - start) / warmdown_frac)
        m = m + t * (end - m)
    return m


def grad_accum_for_step(progress: float, accum: int, half_until: float = 0.0) -> int:
    """Half batch for the first ``half_until`` fraction of the horizon."""
    if half_until > 0 and progress < half_until and accum % 2 == 0:
        return accum // 2
    return accum


def mtp_weights(progress: float, n_targets: int, base: float = 0.5, anneal: float = 0.5) -> tuple:
    """Weights of the extra multi-token-prediction targets at clock fraction ``progress``.  Target k (k = 0 is t+2)
    starts at ``base / 2**k``; the annealing window ``[0, anneal]`` is split into ``n_targets`` equal phases and target k
    falls linearly to zero during phase ``n_targets - 1 - k``, so the farthest target goes first and from ``anneal`` on
    only the next-token loss is left.  With two targets, base 0.5 and anneal 0.5 this is the reference's schedule
    (``mtp_set``, round1/source/train.py:5042-5051): t+3 0.25 -> 0 over [0, 1/4), t+2 0.5 flat then -> 0 over [1/4, 1/2)."""
    if n_targets <= 0:
        return ()
    width = anneal / n_targets
    out = []
    for k in range(n_targets):
        start = width * (n_targets - 1 - k)
        w0 = base / (2 ** k)
        if width <= 0 or progress >= start + width:
            out.append(0.0)
        elif progress <= start:
            out.append(w0)
        else:
            out.append(w0 * (1.0 - (progress - start) / width))
    return tuple(out)


def apply_schedules(optimizer, hyper, step: int, progress: float, tables=None):
    lrm = lr_multiplier(progress, step, hyper.warmup_steps, hyper.warmdown_frac, hyper.final_lr_frac)
    lrm_rows = lr_multiplier(progress, step, hyper.warmup_steps, hyper.rows_warmdown_frac, hyper.rows_final_lr_frac)
    mom = muon_momentum(step, progress, hyper.rows_warmdown_frac)
    for g in optimizer.param_groups:
        g["lr"] = g["initial_lr"] * lrm
        if g["kind"] == "muon":
            g["momentum"] = mom
    return dict(lrm=lrm, lrm_rows=lrm_rows, momentum=mom, table_lr=hyper.table_lr * lrm_rows)
