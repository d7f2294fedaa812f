"""Kernel micro-benchmarks with roofline fractions.

    python -m them_bones_b200.ops.microbench gemm --m 8192 --n 8192 --k 8192 [--pair 1] [--layout nt|nn|tn]
    python -m them_bones_b200.ops.microbench mxgemm --m 65536 --n 5120 --k 1280 [--bn 160|224|256] [--layout nt|tn] [--epi plain|relu2q|relu2qt]
    python -m them_bones_b200.ops.microbench mxquant --rows 65536 --cols 1280
    python -m them_bones_b200.ops.microbench attn_fwd --b 4 --t 2048 --h 10
    python -m them_bones_b200.ops.microbench attn_bwd --b 4 --t 2048 --h 10
    python -m them_bones_b200.ops.microbench norm --rows 65536 --cols 1280
    python -m them_bones_b200.ops.microbench ce --rows 4096 --vocab 65536
    BONES_LIB=them_bones_b200/lib/libbones_b200_prof.so python -m them_bones_b200.ops.microbench mxroles --m 16384 --n 5120 --k 1280 [--epi ...]
    BONES_LIB=them_bones_b200/lib/libbones_b200_prof.so python -m them_bones_b200.ops.microbench attnroles --b 16 --t 2048 --h 10

``mxroles`` / ``attnroles`` need the measuring build of the library (``python -m them_bones_b200.csrc.build --measure``):
they print, per K block or per tile, the clocks each role of the kernel (TMA producer, MMA warp, scale-copy warp,
epilogue / compute warps) spent in each of its waits and in issuing, averaged over the CTAs.

Timing: CUDA events on the launching stream, ``--warmup`` untimed iterations, an L2 flush (a 256 MiB write) between
timed iterations, mean over ``--iters``.  Fractions are against the measured peaks in ``MEASURED_PEAKS.json`` at the
repository root when present (copy bandwidth, cuBLAS bf16 burst), else 6650 GB/s and 1590 TFLOP/s.  ``--iters 1
--warmup 0 --no-flush`` gives a launch list short enough to run under a profiler.
"""
from __future__ import annotations

import argparse
import json
import math
import os

import torch

from . import _lib as L


def peaks():
    root = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    try:
        d = json.load(open(os.path.join(root, "MEASURED_PEAKS.json")))
        return d["hbm_gbs"], d["bf16_tflops"], "measured"
    except (OSError, KeyError, ValueError):
        return 6650.0, 1590.0, "fallback"


def timeit(fn, iters, warmup, flush):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    buf = torch.empty(256 << 20, dtype=torch.uint8, device="cuda") if flush else None
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    total = 0.0
    for _ in range(iters):
        if buf is not None:
            buf.zero_()
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        total += e0.elapsed_time(e1)
    L.check_error_word()
    return total / iters


def roles(a):
    """Role cycle accounting from the measuring build (see the module docstring)."""
    import ctypes
    lib = L.load()
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    prof = torch.zeros(sms * 32, dtype=torch.int64, device="cuda")
    bf = torch.bfloat16
    if a.what == "mxroles":
        from . import mxfp8 as MX
        if not hasattr(lib, "bones_mx2_set_prof"):
            raise SystemExit("mxroles needs the measuring build: python -m them_bones_b200.csrc.build --measure, then BONES_LIB=...")
        m, n, k = a.m, a.n, a.k
        if a.layout == "tn":
            _, _, aq, asf = MX.quant2(torch.randn(k, m, device="cuda", dtype=bf), row=False, col=True, group_c=128)
            _, _, bq, bsf = MX.quant2(torch.randn(k, n, device="cuda", dtype=bf), row=False, col=True, group_c=MX.BN_WGRAD)
            d = torch.zeros(m, n, device="cuda")
            fn = lambda: MX.gemm2(aq, asf, bq, bsf, m, n, k, a_major=1, b_major=1, epi=MX.GE_ACC_F32, out=d, bn=MX.BN_WGRAD)  # noqa: E731
        else:
            bn = a.bn or MX.BN_FWD
            aq, asf, _, _ = MX.quant2(torch.randn(m, k, device="cuda", dtype=bf))
            bq, bsf, _, _ = MX.quant2(torch.randn(n, k, device="cuda", dtype=bf), group_r=bn)
            epi = MX.GE_BF16 if a.epi == "plain" else MX.GE_RELU2
            wq, wt = a.epi in ("relu2q", "relu2qt"), a.epi == "relu2qt"
            fn = lambda: MX.gemm2(aq, asf, bq, bsf, m, n, k, bn=bn, epi=epi, want_q=wq, want_t=wt, dt_group=256)  # noqa: E731
        ms = timeit(fn, a.iters, a.warmup, not a.no_flush)
        lib.bones_mx2_set_prof(ctypes.c_void_p(prof.data_ptr()))
        fn()
        torch.cuda.synchronize()
        lib.bones_mx2_set_prof(ctypes.c_void_p(0))
        pr = prof.view(sms, 32).double()
        lead, peer = pr[0::2].mean(0), pr[1::2].mean(0)
        kb, tiles = float(lead[14]), float(lead[15])
        per = lambda v, d: round(float(v) / max(d, 1.0))  # noqa: E731
        out = {"what": a.what, "shape": [m, n, k], "layout": a.layout, "epi": a.epi, "ms": ms, "tflops": 2.0 * m * n * k / ms / 1e9,
               "k_blocks_per_cta": kb, "tiles_per_cta": tiles,
               "mma_warp_clocks_per_k_block": {"total": per(lead[4], kb), "wait_stage": per(lead[1], kb), "wait_scales": per(lead[2], kb),
                                               "issue": per(lead[16], kb), "loop": per(lead[3], kb), "wait_accumulator": per(lead[0], kb)},
               "producer_clocks_per_k_block": {"wait_empty": per(lead[5], kb), "issue": per(lead[6], kb), "peer_wait_empty": per(peer[5], kb),
                                               "peer_issue": per(peer[6], kb)},
               "scale_copy_clocks_per_k_block": {"wait_stage": per(lead[8], kb), "wait_columns": per(lead[9], kb), "issue": per(lead[10], kb)},
               "epilogue_warp_clocks_per_tile": {"wait_accumulator": per(lead[11], tiles), "drain": per(lead[12], tiles),
                                                 "tmem_load": per(lead[19], tiles), "wait_tma_store": per(lead[20], tiles),
                                                 "maths_and_copy_along_n": per(lead[21], tiles), "copy_along_m": per(lead[22], tiles),
                                                 "read_back_and_stores": per(lead[23], tiles)}}
    else:
        from . import attention_native as AN
        from ..ref import functional as RF
        if not hasattr(lib, "bones_attn_set_prof"):
            raise SystemExit("attnroles needs the measuring build: python -m them_bones_b200.csrc.build --measure, then BONES_LIB=...")
        I, LL, F = ctypes.c_int, ctypes.c_longlong, ctypes.c_float
        b, t, h, d = a.b, a.t, a.h, 128
        ad, m = h * d, b * t
        qkv = torch.randn(m, 3 * ad, device="cuda", dtype=bf)
        cos, sin = RF.rotary_tables(t, d, 10000.0, device="cuda")
        scale = 1.0 / math.sqrt(d)
        qk = AN.rope_qknorm(qkv, cos, sin, t, h, d)
        y, lse = AN.attn_forward(qk, qkv, None, b, t, h, scale, 0)
        dy = torch.randn(m, ad, device="cuda", dtype=bf)
        stats = torch.empty(b, h, t, 2, dtype=torch.float32, device="cuda")
        dqk = torch.empty(m, 2 * ad, dtype=bf, device="cuda")
        dqkv = torch.empty(m, 3 * ad, dtype=bf, device="cuda")
        dv = dqkv[:, 2 * ad:]
        L.call("bones_attn_bwd_stats", L.ptr(dy), L.ptr(y), L.ptr(lse), L.ptr(stats), LL(m), I(t), I(h), L.stream())
        fn = lambda: L.call("bones_attn_bwd_split", L.ptr(qk), L.ptr(qkv), L.ptr(dy), L.ptr(stats), L.ptr(dqk), L.ptr(dv), LL(3 * ad),  # noqa: E731
                            L.ptr(None), I(b), I(t), I(h), F(scale), I(0), L.stream())
        ms = timeit(fn, a.iters, a.warmup, not a.no_flush)
        lib.bones_attn_set_prof(ctypes.c_void_p(prof.data_ptr()))
        fn()
        torch.cuda.synchronize()
        lib.bones_attn_set_prof(ctypes.c_void_p(0))
        pr = prof.view(sms, 32).double().mean(0)
        tiles = float(pr[8])
        per = lambda v: round(float(v) / max(tiles, 1.0))  # noqa: E731
        out = {"what": a.what, "shape": [b, t, h, d], "ms_both_kernels": ms, "dkv_tiles_per_cta": tiles,
               "dkv_mma_warp_clocks_per_tile": {"total": per(pr[7]), "wait_item_kv": per(pr[0]), "wait_q": per(pr[1]), "wait_do": per(pr[2]),
                                                "wait_p_ready": per(pr[3]), "wait_acc_free": per(pr[4]), "wait_ds_ready": per(pr[5]),
                                                "issue": per(pr[6])},
               "dkv_compute_warp_clocks_per_tile": {"total": per(pr[17]), "wait_stats": per(pr[10]), "wait_s": per(pr[11]), "p": per(pr[12]),
                                                    "wait_dp": per(pr[13]), "ds": per(pr[14]), "wait_done": per(pr[15]), "drain": per(pr[16])},
               "dkv_producer_clocks_per_tile": {"waits": per(pr[20]), "issue": per(pr[21])}}
    print(json.dumps(out))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("what", choices=["gemm", "mxgemm", "mxquant", "attn_fwd", "attn_bwd", "norm", "ce", "mxroles", "attnroles"])
    ap.add_argument("--m", type=int, default=8192)
    ap.add_argument("--n", type=int, default=8192)
    ap.add_argument("--k", type=int, default=8192)
    ap.add_argument("--pair", type=int, default=1)
    ap.add_argument("--layout", default="nt")
    ap.add_argument("--bn", type=int, default=0, help="mxgemm: pair tile N (0: the operator default)")
    ap.add_argument("--epi", default="plain", help="mxgemm: plain | relu2q (+ copy quantised along N) | relu2qt (+ along M too)")
    ap.add_argument("--b", type=int, default=4)
    ap.add_argument("--t", type=int, default=2048)
    ap.add_argument("--h", type=int, default=10)
    ap.add_argument("--rows", type=int, default=65536)
    ap.add_argument("--cols", type=int, default=1280)
    ap.add_argument("--vocab", type=int, default=65536)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--capped", type=int, default=1, help="ce: 1 = logits already soft-capped by the GEMM epilogue (the training path)")
    ap.add_argument("--no-flush", action="store_true")
    a = ap.parse_args()
    hbm, tf, src = peaks()
    bf = torch.bfloat16
    out = {"what": a.what, "peaks": src}
    torch.manual_seed(0)
    if a.what in ("mxroles", "attnroles"):
        return roles(a)
    if a.what == "gemm":
        m, n, k = a.m, a.n, a.k
        if a.layout == "nt":
            x, w, d = torch.randn(m, k, device="cuda", dtype=bf), torch.randn(n, k, device="cuda", dtype=bf), torch.empty(m, n, device="cuda", dtype=bf)
            fn = lambda: L.gemm(x, w, d, m=m, n=n, k=k, lda=k, ldb=k, ldd=n, pair=bool(a.pair))  # noqa: E731
        elif a.layout == "nn":
            x, w, d = torch.randn(m, k, device="cuda", dtype=bf), torch.randn(k, n, device="cuda", dtype=bf), torch.empty(m, n, device="cuda", dtype=bf)
            fn = lambda: L.gemm(x, w, d, m=m, n=n, k=k, lda=k, ldb=n, ldd=n, b_major=1, pair=bool(a.pair))  # noqa: E731
        else:
            x, w, d = torch.randn(k, m, device="cuda", dtype=bf), torch.randn(k, n, device="cuda", dtype=bf), torch.zeros(m, n, device="cuda")
            fn = lambda: L.gemm(x, w, d, m=m, n=n, k=k, lda=m, ldb=n, ldd=n, a_major=1, b_major=1, epi=L.EPI_ACC_F32, pair=bool(a.pair))  # noqa: E731
        ms = timeit(fn, a.iters, a.warmup, not a.no_flush)
        fl = 2.0 * m * n * k
        out.update(shape=[m, n, k], layout=a.layout, pair=a.pair, ms=ms, tflops=fl / ms / 1e9, frac_of_bf16_peak=fl / ms / 1e9 / tf)
    elif a.what == "mxgemm":
        from . import mxfp8 as MX
        m, n, k = a.m, a.n, a.k
        if a.layout == "tn":          # weight gradient: contraction over the token axis, both operands MN-major
            _, _, aq, asf = MX.quant2(torch.randn(k, m, device="cuda", dtype=bf), row=False, col=True, group_c=128)
            _, _, bq, bsf = MX.quant2(torch.randn(k, n, device="cuda", dtype=bf), row=False, col=True, group_c=MX.BN_WGRAD)
            d = torch.zeros(m, n, device="cuda")
            fn = lambda: MX.gemm2(aq, asf, bq, bsf, m, n, k, a_major=1, b_major=1, epi=MX.GE_ACC_F32, out=d, bn=MX.BN_WGRAD)  # noqa: E731
        else:
            bn = a.bn or MX.BN_FWD
            aq, asf, _, _ = MX.quant2(torch.randn(m, k, device="cuda", dtype=bf))
            bq, bsf, _, _ = MX.quant2(torch.randn(n, k, device="cuda", dtype=bf), group_r=bn)
            d = torch.empty(m, n, device="cuda", dtype=bf)
            dq = torch.empty(m, n, device="cuda", dtype=torch.uint8)
            dsf = torch.zeros(MX.sf2_bytes(m, n, 128), device="cuda", dtype=torch.uint8)
            dt = torch.empty(m, n, device="cuda", dtype=torch.uint8)
            dtsf = torch.zeros(MX.sf2_bytes(n, m, 256), device="cuda", dtype=torch.uint8)
            import ctypes
            I, LL, F = ctypes.c_int, ctypes.c_longlong, ctypes.c_float
            epi = MX.GE_BF16 if a.epi == "plain" else MX.GE_RELU2
            wq, wt = a.epi in ("relu2q", "relu2qt"), a.epi == "relu2qt"
            fn = lambda: L.call("bones_gemm_mxfp8_pair", L.ptr(aq), L.ptr(asf), L.ptr(bq), L.ptr(bsf), L.ptr(d), L.ptr(None),  # noqa: E731
                                L.ptr(dq if wq else None), L.ptr(dsf if wq else None), I(128), L.ptr(dt if wt else None),
                                L.ptr(dtsf if wt else None), I(256), I(m), I(n), I(k), I(1), LL(k), LL(k), LL(n), LL(0), LL(0), LL(0),
                                LL(0), LL(0), I(0), I(0), I(epi), F(1.0), F(1.0), I(bn), I(0), I(0), L.stream())
        ms = timeit(fn, a.iters, a.warmup, not a.no_flush)
        fl = 2.0 * m * n * k
        out.update(shape=[m, n, k], layout=a.layout, bn=a.bn, epi=a.epi, ms=ms, tflops=fl / ms / 1e9, frac_of_bf16_peak=fl / ms / 1e9 / tf)
    elif a.what == "mxquant":
        from . import mxfp8 as MX
        x = torch.randn(a.rows, a.cols, device="cuda", dtype=bf)
        ms = timeit(lambda: MX.quant2(x, col=True), a.iters, a.warmup, not a.no_flush)
        by = 4.0 * x.numel()                                    # one bf16 read, two fp8 writes
        out.update(shape=[a.rows, a.cols], ms=ms, gbs=by / ms / 1e6, frac_of_hbm_peak=by / ms / 1e6 / hbm)
    elif a.what in ("attn_fwd", "attn_bwd"):
        from . import attention_bwd as AB
        from . import attention_native as AN
        from ..ref import functional as RF
        b, t, h, d = a.b, a.t, a.h, 128
        qkv = torch.randn(b * t, 3 * h * d, device="cuda", dtype=bf)
        cos, sin = RF.rotary_tables(t, d, 10000.0, device="cuda")
        scale = 1.0 / math.sqrt(d)
        qk = AN.rope_qknorm(qkv, cos, sin, t, h, d)
        y, lse = AN.attn_forward(qk, qkv, None, b, t, h, scale, 0)
        fl = 4.0 * b * h * t * t * d / 2                      # causal: half the square
        if a.what == "attn_fwd":
            ms = timeit(lambda: AN.attn_forward(qk, qkv, None, b, t, h, scale, 0), a.iters, a.warmup, not a.no_flush)
        else:
            dy = torch.randn(b * t, h * d, device="cuda", dtype=bf)
            ms = timeit(lambda: AB.backward(dy, qkv, qk, y, lse, cos, sin, None, b, t, h, d, scale, 0), a.iters, a.warmup,
                        not a.no_flush)
            fl *= 2.5
        out.update(shape=[b, t, h, d], ms=ms, tflops=fl / ms / 1e9, frac_of_bf16_peak=fl / ms / 1e9 / tf)
    elif a.what == "norm":
        from . import cuda as C
        x = torch.randn(a.rows, a.cols, device="cuda", dtype=bf)
        x0 = torch.randn_like(x)
        one, small = torch.ones(1, device="cuda"), torch.full((1,), 0.05, device="cuda")
        with torch.no_grad():
            ms = timeit(lambda: C.resid_mix_norm(x, x0, one, small), a.iters, a.warmup, not a.no_flush)
        by = 4.0 * x.numel() * 2                                # two reads, two writes
        out.update(shape=[a.rows, a.cols], ms=ms, gbs=by / ms / 1e6, frac_of_hbm_peak=by / ms / 1e6 / hbm)
    else:
        import ctypes
        rows, v = a.rows, a.vocab
        lg = torch.randn(rows, v, device="cuda", dtype=bf)
        tg = torch.randint(0, v, (rows,), device="cuda")
        nll = torch.empty(rows, device="cuda")
        nv = torch.full((1,), float(rows), device="cuda")
        fn = lambda: L.call("bones_softcap_ce", L.ptr(lg), ctypes.c_longlong(v), L.ptr(tg), ctypes.c_int(v),  # noqa: E731
                            ctypes.c_float(15.0), L.ptr(nll), L.ptr(lg), L.ptr(None), L.ptr(nv), ctypes.c_float(1.0),
                            ctypes.c_int(rows), ctypes.c_int(a.capped), L.ptr(None), L.ptr(None), L.ptr(None), L.ptr(None), L.ptr(None),
                            ctypes.c_float(0.0), L.stream())
        ms = timeit(fn, a.iters, a.warmup, not a.no_flush)
        by = 2.0 * lg.numel() * 2                               # one read, one write (the row stays in registers)
        out.update(shape=[rows, v], capped=a.capped, ms=ms, gbs=by / ms / 1e6, frac_of_hbm_peak=by / ms / 1e6 / hbm)
    print(json.dumps(out))


if __name__ == "__main__":
    main()
