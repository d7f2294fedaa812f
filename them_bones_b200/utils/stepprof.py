"""Kernel breakdown of one training step of the dense benchmark model (20 layers x 1280, vocabulary 65536, sequence 2048).

    python -m them_bones_b200.utils.stepprof [--total-batch 524288] [--device-batch 64] [--mlp mxfp8] [--attn-proj bf16] [--moe]
    python -m torch.distributed.run --nproc-per-node N --master-addr 127.0.0.1 -m them_bones_b200.utils.stepprof

Builds the ``Trainer`` as ``bench.py`` does, runs three warm-up steps, then one step under ``torch.profiler`` (CUDA
activities only) and prints, on rank 0, the device time per kernel name and the kernels of the step-boundary chain
(everything after the last backward kernel: gradient reduction, optimizer, weight publication) with the wall span they
cover.  Times taken under the profiler are for shares, not for throughput.
"""
from __future__ import annotations

import argparse
import collections
import time

import torch


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--total-batch", type=int, default=524288)
    ap.add_argument("--device-batch", type=int, default=64)
    ap.add_argument("--depth", type=int, default=20)
    ap.add_argument("--mlp", default="mxfp8")
    ap.add_argument("--attn-proj", default="bf16")
    ap.add_argument("--top", type=int, default=30)
    ap.add_argument("--moe", action="store_true", help="the MoE model: 16 experts, top-2, every MLP from layer 2 on")
    a = ap.parse_args()
    from ..config import GPTConfig, Hyper, micro_batch_for, moe_capacity_for
    from ..data.synth import SynthLoader
    from ..runtime import init_runtime
    from ..trainer import Trainer
    rt = init_runtime("cuda")
    kw = {}
    if a.moe:
        kw = dict(moe_layers=tuple(range(2, a.depth)), moe_experts=16, moe_topk=2, moe_hidden=2560,
                  moe_capacity=moe_capacity_for(1.25, 2048, 2, 16), moe_aux=0.01)
    cfg = GPTConfig(sequence_len=2048, vocab_size=65536, n_layer=a.depth, n_head=10, n_embd=1280, head_dim=128, doc_mask=True,
                    mlp_precision=a.mlp, attn_proj_precision=a.attn_proj, **kw)
    h = Hyper()
    h.total_batch, h.device_batch = a.total_batch, micro_batch_for(a.total_batch, rt.world, a.device_batch, 2048)
    tr = Trainer(cfg, h, rt)
    ld = SynthLoader(65536, 2048, tr.local_windows, rank=rt.rank, seed=0, pin=True, shard_of=rt.world)
    x, y = ld.next_step()
    x, y = x.to(rt.device), y.to(rt.device)
    for _ in range(3):
        tr.train_step(x, y)
    torch.cuda.synchronize()
    if rt.ddp:
        torch.distributed.barrier()
    t0 = time.time()
    tr.train_step(x, y)
    torch.cuda.synchronize()
    wall = (time.time() - t0) * 1e3
    from torch.profiler import ProfilerActivity, profile
    with profile(activities=[ProfilerActivity.CUDA]) as prof:
        tr.train_step(x, y)
        torch.cuda.synchronize()
    if rt.rank == 0:
        print(f"world {rt.world}  device batch {tr.device_batch}  micro-steps {tr.grad_accum}  wall {wall:.1f} ms per step (no profiler)")
        evs = [e for e in prof.events() if e.device_type.name == "CUDA"]
        agg = collections.defaultdict(lambda: [0.0, 0])
        for e in evs:
            agg[e.name][0] += e.device_time
            agg[e.name][1] += 1
        rows = sorted(agg.items(), key=lambda kv: -kv[1][0])
        tot = sum(v[0] for _, v in rows)
        print(f"kernel time {tot / 1e3:.1f} ms in {len(evs)} launches")
        for k, (t, c) in rows[:a.top]:
            print(f"{t / 1e3:9.2f} ms {100 * t / tot:5.1f} % x{c:5d}  {k[:96]}")
        evs.sort(key=lambda e: e.time_range.start)
        marks = [i for i, e in enumerate(evs) if "attn_bwd" in e.name or "rope_qknorm_bwd" in e.name or "scatter_add_rows" in e.name]
        tail = evs[marks[-1] + 1:] if marks else []
        if tail:
            span = (tail[-1].time_range.end - tail[0].time_range.start) / 1e3
            busy = sum(e.device_time for e in tail) / 1e3
            print(f"step-boundary chain: {len(tail)} kernels, span {span:.2f} ms, busy {busy:.2f} ms")
            agg2 = collections.defaultdict(lambda: [0.0, 0])
            for e in tail:
                agg2[e.name][0] += e.device_time
                agg2[e.name][1] += 1
            for k, (t, c) in sorted(agg2.items(), key=lambda kv: -kv[1][0])[:14]:
                print(f"   {t / 1e3:8.3f} ms x{c:4d}  {k[:96]}")
    if rt.ddp:
        torch.distributed.barrier()
        torch.distributed.destroy_process_group()


if __name__ == "__main__":
    main()
