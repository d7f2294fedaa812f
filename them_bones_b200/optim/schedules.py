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


def apply_schedules(optimizer, hyper, step: int, progress: float, tables=None):
    lrm = lr_multiplier(progress, step, hyper.warmup_steps, hyper.warmdown_frac, hyper.final_lr_frac)
    lrm_rows = lr_multiplier(progress, step, hyper.warmup_steps, hyper.rows_warmdown_frac, hyper.rows_final_lr_frac)
    mom = muon_momentum(step, progress, hyper.rows_warmdown_frac)
    for g in optimizer.param_groups:
        g["lr"] = g["initial_lr"] * lrm
        if g["kind"] == "muon":
            g["momentum"] = mom
    return dict(lrm=lrm, lrm_rows=lrm_rows, momentum=mom, table_lr=hyper.table_lr * lrm_rows)
