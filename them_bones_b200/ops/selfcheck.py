"""First-call self-check: every native op against its plain-PyTorch statement on small live tensors, before the clock
starts (reference: the first-call on-device checks ``lossk__multi_selfcheck`` round1/source/train.py:4948,
``mixk__selfcheck`` :7395, and the rule that a kernel which does not apply raises on the device).

``run()`` returns ``{name: relative error}`` and raises ``RuntimeError`` when an error exceeds its tolerance or a kernel
reported a bounded-wait expiry.  ``train.py`` calls it when ``BONES_SELFCHECK=1``.
"""
from __future__ import annotations

import torch

from .. import ops
from ..ref import functional as RF


def _rel(a, b) -> float:
    a, b = a.detach().float(), b.detach().float()
    return float((a - b).norm() / b.norm().clamp_min(1e-12))


def _both(fn):
    """Run ``fn`` on the native path and on the reference path (same inputs, fresh autograd leaves)."""
    was = ops.reference_path()
    try:
        ops.set_reference_path(False)
        nat = fn()
        ops.set_reference_path(True)
        ref = fn()
    finally:
        ops.set_reference_path(was)
    return nat, ref


def run(device="cuda", seed: int = 0, verbose: bool = False) -> dict:
    from . import _lib as L
    if not torch.cuda.is_available():
        raise RuntimeError("the self-check compares the CUDA kernels with the PyTorch path: no GPU here")
    g = torch.Generator(device=device).manual_seed(seed)
    bf = torch.bfloat16

    def rnd(*shape, scale=1.0):
        return (torch.randn(*shape, device=device, generator=g) * scale).to(bf)

    out, tol = {}, {}

    def check(name, nat, ref, t):
        for i, (a, b) in enumerate(zip(nat, ref)):
            out[f"{name}[{i}]"] = _rel(a, b)
            tol[f"{name}[{i}]"] = t

    m, c, hdim, heads, t_len, vocab = 512, 256, 128, 2, 256, 8192
    # linear (+ residual), fused qkv, MLP: forward and the three gradients
    x, w, r = rnd(m, c), rnd(3 * c, c, scale=0.06), rnd(m, 3 * c)

    def lin():
        xx, ww = x.clone().requires_grad_(), w.clone().requires_grad_()
        y = ops.linear(xx, ww, residual=r)
        y.float().square().sum().backward()
        return y, xx.grad, ww.grad
    check("linear", *_both(lin), 3e-2)
    wf, wp = rnd(4 * c, c, scale=0.06), rnd(c, 4 * c, scale=0.03)

    def mlp():
        xx, a, b = x.clone().requires_grad_(), wf.clone().requires_grad_(), wp.clone().requires_grad_()
        y = ops.mlp(xx, a, b, residual=x)
        y.float().square().sum().backward()
        return y, xx.grad, a.grad, b.grad
    check("mlp", *_both(mlp), 5e-2)
    # norms
    x0, ga, gb = rnd(m, c), torch.tensor([0.9], device=device), torch.tensor([0.1], device=device)

    def norms():
        xx, yy = x.clone().requires_grad_(), x0.clone().requires_grad_()
        a, b = ga.clone().requires_grad_(), gb.clone().requires_grad_()
        xm, xn = ops.resid_mix_norm(xx, yy, a, b)
        xp, xq = ops.norm_split(xm)
        (xn.float() * 0.5 + xq.float() + xp.float() * 0.25).square().sum().backward()
        return xm, xn, xx.grad, yy.grad
    check("norms", *_both(norms), 3e-2)
    # attention with document starts and a window
    qkv = rnd(2, t_len, 3 * heads * hdim)
    cos, sin = RF.rotary_tables(t_len, hdim, 100000.0, device=device)
    ids = torch.randint(1, 100, (2, t_len), device=device, generator=g)
    ids[:, 0] = 0
    ids[0, 100] = 0
    ds = RF.doc_start_positions(ids, 0)

    def attn():
        q = qkv.clone().requires_grad_()
        y = ops.attention(q, cos, sin, heads, hdim, 0.11, ds, 128)
        (y.float() * torch.linspace(-1, 1, y.shape[-1], device=device)).sum().backward()
        return y, q.grad
    check("attention", *_both(attn), 5e-2)
    # loss head with two auxiliary targets
    h, wl = rnd(m, c), rnd(vocab, c, scale=0.05)
    tg = torch.randint(0, vocab, (m,), device=device, generator=g)
    tg[::17] = -1
    t2 = torch.roll(tg, -1)
    aw = torch.full((m,), 0.5 / m, device=device)

    def head():
        hh, ww = h.clone().requires_grad_(), wl.clone().requires_grad_()
        loss = ops.lmhead_loss(hh, ww, tg, vocab, 15.0, aux=[(t2, aw)])
        loss.backward()
        return loss.reshape(1), hh.grad, ww.grad
    check("loss_head", *_both(head), 5e-2)
    torch.cuda.synchronize()
    L.check_error_word()
    bad = {k: v for k, v in out.items() if not (v <= tol[k])}
    if verbose or bad:
        for k, v in out.items():
            print(f"selfcheck {k:16s} rel err {v:.3e} (tolerance {tol[k]:.0e})", flush=True)
    if bad:
        raise RuntimeError(f"native kernels disagree with the PyTorch path: {bad}")
    return out
