"""ctypes binding of the native library ``them_bones_b200/lib/libbones_b200.so``.

The library is plain C ABI: every entry point takes raw device pointers, sizes and the CUDA stream, launches
asynchronously and returns 0 or an error code.  It is built in-tree by ``csrc/build.py`` (nvcc, sm_100a) and is
required on a GPU: a missing or unloadable library raises here rather than letting a GPU run continue on a fallback.
"""
from __future__ import annotations

import ctypes
import os

import torch

_LIB = None
DEBUG_BOUNDS = os.environ.get("BONES_DEBUG_BOUNDS", "0") not in ("0", "", "false")
# BONES_LIB: path of another build of the library (for instance one compiled with a measuring define)
_PATH = os.environ.get("BONES_LIB") or os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "lib",
                                                    "libbones_b200_dbg.so" if DEBUG_BOUNDS else "libbones_b200.so")


def lib_path() -> str:
    return _PATH


def load():
    global _LIB
    if _LIB is None:
        if not os.path.exists(_PATH):
            raise RuntimeError(f"native library missing: {_PATH}; run `python -m them_bones_b200.csrc.build` "
                               "(or __graft_entry__.build()) first")
        _LIB = ctypes.CDLL(_PATH)
    return _LIB


def available() -> bool:
    try:
        load()
        return True
    except (RuntimeError, OSError):
        return False


def ptr(t):
    return ctypes.c_void_p(0 if t is None else t.data_ptr())


def stream():
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


_I, _L, _F = ctypes.c_int, ctypes.c_longlong, ctypes.c_float


LAUNCHES = [0]        # native kernel launches issued by this process (each entry point launches one kernel)


def call(name: str, *args):
    LAUNCHES[0] += 1
    rc = getattr(load(), name)(*args)
    if rc != 0:
        raise RuntimeError(f"{name} failed with code {rc}")


def check_error_word():
    """Raises if any kernel on the current device gave up on a bounded wait since the last check.  Synchronises."""
    rc = load().bones_error_read_clear()
    if rc != 0:
        raise RuntimeError(f"a native kernel reported error code {rc} (bounded wait expired or bad argument)")
    if DEBUG_BOUNDS:
        hits = bounds_hits()
        if hits:
            raise RuntimeError(f"debug-bounds build: out-of-range indices were caught and skipped: {hits}")


def bounds_hits() -> dict:
    """Debug-bounds library only: ``{source file: (count, offending index, source line)}`` of the index checks that
    failed since the last call (read and cleared; synchronises)."""
    out = {}
    lib = load()
    for tu in ("elementwise", "comm", "tables"):
        fn = getattr(lib, f"bones_bounds_hits_{tu}", None)
        if fn is None:
            continue
        last = (ctypes.c_longlong * 2)()
        n = fn(last)
        if n:
            out[tu] = (int(n), int(last[0]), int(last[1]))
    return out


EPI_BF16, EPI_BF16_RES, EPI_RELU2, EPI_ACC_F32, EPI_MUL_2SQRT, EPI_F32, EPI_F32_RES, EPI_SOFTCAP = range(8)


PAIR_MODE = os.environ.get("BONES_GEMM_PAIR", "auto")      # auto | 0 | 1


def gemm(a, b, d, *, m, n, k, lda, ldb, ldd, a_major=0, b_major=0, epi=EPI_BF16, r=None, ldr=0, alpha=1.0, beta=1.0,
         batch=1, stride_a=0, stride_b=0, stride_d=0, stride_r=0, force_bn=0, splits=0, pair=None, d_ptr=None, atomic=False):
    """``d = epilogue(alpha * a @ b^T, r)``; see csrc/gemm_bf16.cu for operand layouts.  Large problems run on CTA
    pairs (csrc/gemm_bf16_2cta.cu: 256 x 256 tiles, one third less L2 traffic per flop); small ones on single CTAs."""
    if pair is None:
        if PAIR_MODE == "auto":
            tiles = -(-m // 256) * -(-n // 256) * batch
            # few output tiles still fill the pairs when a long K is split (weight gradients)
            pair = force_bn == 0 and m >= 256 and n >= 256 and (tiles >= 37 or (epi == EPI_ACC_F32 and k >= 8192 * 37 // tiles))
        else:
            pair = PAIR_MODE == "1" and force_bn == 0
    # d_ptr: raw device address used instead of ``d`` (e.g. the same buffer in another GPU's memory); atomic: fp32
    # accumulation by vector atomics even without split-K, for outputs several GPUs add into at once
    dp = ptr(d) if d_ptr is None else ctypes.c_void_p(int(d_ptr))
    if pair:
        call("bones_gemm_bf16_pair", ptr(a), ptr(b), dp, ptr(r), _I(m), _I(n), _I(k), _I(batch), _L(lda), _L(ldb),
             _L(ldd), _L(ldr), _L(stride_a), _L(stride_b), _L(stride_d), _L(stride_r), _I(a_major), _I(b_major), _I(epi),
             _F(alpha), _F(beta), _I(splits), _I(int(atomic)), stream())
        return
    call("bones_gemm_bf16", ptr(a), ptr(b), dp, ptr(r), _I(m), _I(n), _I(k), _I(batch), _L(lda), _L(ldb), _L(ldd),
         _L(ldr), _L(stride_a), _L(stride_b), _L(stride_d), _L(stride_r), _I(a_major), _I(b_major), _I(epi), _F(alpha),
         _F(beta), _I(force_bn), _I(splits), _I(int(atomic)), stream())
