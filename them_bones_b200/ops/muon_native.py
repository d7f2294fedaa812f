"""Muon's Newton-Schulz iteration on the tcgen05 GEMM (batched over the matrices of a shape group).

Polar-Express iteration (coefficients and tall/wide forms: reference round2/source/train.py:11755-11761, :11880-11888;
its on-chip kernel: round2/source/kernels/nki_nsk.py): tall matrices iterate on ``G = X^T X`` and wide ones on
``G = X X^T``; ``B = b G + c G^2``; ``X' = a X + X B`` (tall) or ``a X + B X`` (wide).  ``G`` and ``B`` are symmetric, so
every product is issued as a K-major or MN-major operand view of the same buffers (no transposes): three batched GEMM
launches per iteration with the ``alpha*acc + beta*R`` epilogue doing the polynomial.
"""
from __future__ import annotations

import torch

from ..ref.functional import POLAR_EXPRESS_COEFFS
from . import COUNTS
from . import _lib as L


def newton_schulz(x: torch.Tensor, steps: int = 5) -> torch.Tensor:
    """``x [k, r, c]`` bf16, Frobenius-normalised.  Returns the orthogonalised stack (bf16, new tensor)."""
    assert x.dtype == torch.bfloat16 and x.is_contiguous()
    k, r, c = x.shape
    if r % 8 or c % 8:       # tiny matrices (a 16 x d router): not worth a tensor-core tile, and below the TMA alignment
        from ..ref.functional import newton_schulz as ns_ref
        return ns_ref(x, steps)
    tall = r > c
    n = c if tall else r
    g = torch.empty(k, n, n, dtype=torch.bfloat16, device=x.device)
    b = torch.empty_like(g)
    cur, nxt = x, torch.empty_like(x)
    for ca, cb, cc in POLAR_EXPRESS_COEFFS[:steps]:
        if tall:     # G = X^T X: both operands are MN-major views of X (contraction over rows)
            L.gemm(cur, cur, g, m=c, n=c, k=r, lda=c, ldb=c, ldd=c, a_major=1, b_major=1, batch=k, stride_a=r * c,
                   stride_b=r * c, stride_d=n * n)
        else:        # G = X X^T
            L.gemm(cur, cur, g, m=r, n=r, k=c, lda=c, ldb=c, ldd=r, batch=k, stride_a=r * c, stride_b=r * c, stride_d=n * n)
        # B = cb * G + cc * G G   (G symmetric: G G = G G^T)
        L.gemm(g, g, b, m=n, n=n, k=n, lda=n, ldb=n, ldd=n, epi=L.EPI_BF16_RES, r=g, ldr=n, alpha=cc, beta=cb, batch=k,
               stride_a=n * n, stride_b=n * n, stride_d=n * n, stride_r=n * n)
        if tall:     # X' = ca * X + X B   (B symmetric: X B = X B^T)
            L.gemm(cur, b, nxt, m=r, n=c, k=c, lda=c, ldb=c, ldd=c, epi=L.EPI_BF16_RES, r=cur, ldr=c, alpha=1.0, beta=ca,
                   batch=k, stride_a=r * c, stride_b=n * n, stride_d=r * c, stride_r=r * c)
        else:        # X' = ca * X + B X   (X as an MN-major operand: contraction over its rows)
            L.gemm(b, cur, nxt, m=r, n=c, k=r, lda=r, ldb=c, ldd=c, b_major=1, epi=L.EPI_BF16_RES, r=cur, ldr=c, alpha=1.0,
                   beta=ca, batch=k, stride_a=n * n, stride_b=r * c, stride_d=r * c, stride_r=r * c)
        cur, nxt = nxt, (cur if cur is not x else torch.empty_like(x))
        COUNTS["ns_gemm"] += 3
    return cur


@torch.no_grad()
def muon_finish(g, w, second, *, beta2, lr, wd):
    """NorMuon second-moment rescale (keeps the Frobenius norm), cautious weight decay and the master update, on the
    owner's fp32 master ``w [k, r, c]`` (reference: round2/source/train.py:11890-11905).  Two native passes over the
    stack (``csrc/muon.cu``: line statistics, update); the arithmetic on the ``k * r`` or ``k * c`` line values between
    them is PyTorch."""
    import ctypes
    k, r, c = g.shape
    lr_eff = lr * max(1.0, r / c) ** 0.5
    by_row = r >= c
    if not (g.is_cuda and g.dtype == torch.bfloat16 and w.dtype == torch.float32 and c % 2 == 0 and g.is_contiguous()
            and w.is_contiguous()):
        return _muon_finish_torch(g, w, second, beta2=beta2, lr=lr, wd=wd)
    _I, _F = ctypes.c_int, ctypes.c_float
    v_mean = torch.empty(second.shape, dtype=torch.float32, device=g.device)
    L.call("bones_muon_linesq", L.ptr(g), L.ptr(v_mean), _I(k), _I(r), _I(c), _I(int(by_row)), L.stream())
    n_red = c if by_row else r
    v_norm = (v_mean.sum(dim=(-2, -1), keepdim=True) * n_red).sqrt()
    second.lerp_(v_mean, 1 - beta2)
    step_size = second.clamp_min(1e-10).rsqrt()
    v_norm_new = ((v_mean * n_red) * step_size.square()).sum(dim=(-2, -1), keepdim=True).sqrt()
    line_scale = (step_size * (v_norm / v_norm_new.clamp_min(1e-10))).contiguous()
    L.call("bones_muon_apply", L.ptr(g), L.ptr(w), L.ptr(line_scale), _I(k), _I(r), _I(c), _I(int(by_row)), _F(lr_eff),
           _F(lr_eff * wd), L.stream())
    COUNTS["muon_finish"] += 1
    return w


@torch.no_grad()
def _muon_finish_torch(g, w, second, *, beta2, lr, wd):
    r, c = g.shape[-2:]
    lr_eff = lr * max(1.0, r / c) ** 0.5
    red_dim = -1 if r >= c else -2
    gf = g.float()
    v_mean = gf.square().mean(dim=red_dim, keepdim=True)
    n_red = g.size(red_dim)
    v_norm = (v_mean.sum(dim=(-2, -1), keepdim=True) * n_red).sqrt()
    second.lerp_(v_mean, 1 - beta2)
    step_size = second.clamp_min(1e-10).rsqrt()
    scaled = (v_mean * n_red) * step_size.square()
    v_norm_new = scaled.sum(dim=(-2, -1), keepdim=True).sqrt()
    gf = gf * (step_size * (v_norm / v_norm_new.clamp_min(1e-10)))
    mask = (gf * w) >= 0
    w.sub_(lr_eff * gf + lr_eff * wd * w * mask)
    return w
