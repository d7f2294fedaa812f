"""Secondary benchmarks (the headline benchmark is ``bench.py``): MoE training, MoE + hashed tables, inference.

    python bench_extra.py --what moe    [--gpus N under torch.distributed.run] --steps 2 --warmup 2
    python bench_extra.py --what full   --table-rows 4194304          (MoE + bigram/trigram tables)
    python bench_extra.py --what os1    --os1-rows 16777216            (dense decoder + output-side table)
    python bench_extra.py --what infer  --requests 256 --decode-batch 64 --new-tokens 128

Same timing rules as ``bench.py`` (CUDA events, max over ranks, warm-up first).  Prints one JSON line on rank 0.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--what", default="moe", choices=["moe", "full", "os1", "infer"])
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=2)
    ap.add_argument("--warmup", type=int, default=2)
    ap.add_argument("--depth", type=int, default=20)
    ap.add_argument("--total-batch", type=int, default=524288)
    ap.add_argument("--device-batch", type=int, default=8)
    ap.add_argument("--table-rows", type=int, default=1 << 22)
    ap.add_argument("--os1-rows", type=int, default=1 << 24)
    ap.add_argument("--requests", type=int, default=256)
    ap.add_argument("--decode-batch", type=int, default=64)
    ap.add_argument("--new-tokens", type=int, default=128)
    a = ap.parse_args()

    import torch
    import torch.distributed as dist

    from them_bones_b200 import ops
    from them_bones_b200.config import GPTConfig, Hyper, moe_capacity_for
    from them_bones_b200.data.synth import SynthLoader
    from them_bones_b200.ops import _lib
    from them_bones_b200.runtime import init_runtime, max_over_ranks

    rt = init_runtime("cuda")
    kw = dict(sequence_len=2048, vocab_size=65536, n_layer=a.depth, n_head=10, n_embd=1280, head_dim=128, doc_mask=True)
    if a.what in ("moe", "full", "infer"):
        kw.update(moe_layers=tuple(range(2, a.depth)), moe_experts=16, moe_topk=2, moe_hidden=2560,
                  moe_capacity=moe_capacity_for(1.25, 2048, 2, 16), moe_aux=0.01)
    if a.what == "full":
        kw.update(table_orders=(2, 3), table_rows=a.table_rows)
    if a.what == "os1":
        kw.update(os1_rows=a.os1_rows)
    cfg = GPTConfig(**kw)

    def barrier():
        if rt.ddp:
            dist.barrier()
        torch.cuda.synchronize()

    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    if a.what in ("moe", "full", "os1"):
        from them_bones_b200.trainer import Trainer
        hy = Hyper()
        hy.total_batch, hy.device_batch = a.total_batch, a.device_batch
        tr = Trainer(cfg, hy, rt, horizon_steps=1000)
        ld = SynthLoader(cfg.vocab_size, 2048, tr.local_windows, rank=rt.rank, seed=1, pin=True)
        batches = [ld.next_step() for _ in range(2)]
        for i in range(a.warmup):
            tr.train_step(*batches[i % 2])
        barrier()
        e0.record()
        for i in range(a.steps):
            loss = tr.train_step(*batches[i % 2])
        e1.record()
        barrier()
        _lib.check_error_word()
        ms = max_over_ranks(e0.elapsed_time(e1), rt)
        if rt.rank == 0:
            print(json.dumps({"metric": "train tokens/sec (device-timed, max over ranks, host->device copies included)",
                              "what": a.what, "value": a.steps * tr.total_batch / (ms / 1e3), "unit": "tokens/s",
                              "n_gpus": rt.world, "ms_per_step": ms / a.steps, "loss": float(loss),
                              "config": {"model": (f"dense {a.depth}Lx1280 + output table {a.os1_rows} rows x 128, order 16" if a.what == "os1" else
                                                   f"moe 16e top-2 {a.depth}Lx1280" + (f" + tables {a.table_rows} rows" if a.what == "full" else "")),
                                         "global_batch": tr.total_batch, "experts_per_gpu": 16 // rt.world,
                                         "fused_comm": tr.comm is not None},
                              "os1_stats": tr.os1.stats if tr.os1 is not None else None,
                              "native_ops": dict(ops.COUNTS), "moe_stats": (tr.last_moe_stats.float().mean(0)[:3].tolist()
                                                                            if tr.last_moe_stats is not None else None)}), flush=True)
    else:
        from them_bones_b200.models.gpt import GPT
        from them_bones_b200.utils.decode import greedy_decode
        from them_bones_b200.utils.evalbpb import score_continuations
        torch.manual_seed(0)
        cfg_i = GPTConfig(**{**kw, "moe_layers": ()})            # dense scoring replica per rank (all weights local)
        model = GPT(cfg_i)
        model.init_weights()
        model = model.cuda().cast_compute(torch.bfloat16).eval()
        g = torch.Generator().manual_seed(rt.rank)
        n, bsz = a.requests, 8
        toks = torch.randint(1, 65536, (n, 2048), generator=g)
        toks[:, 0] = 0
        total = torch.randint(512, 2049, (n,), generator=g)
        cont = torch.randint(1, 65, (n,), generator=g)
        ctx = total - cont
        with torch.no_grad():
            score_continuations(model, toks[:bsz].cuda(), ctx[:bsz].cuda(), total[:bsz].cuda())
            barrier()
            e0.record()
            for i in range(0, n, bsz):
                s = score_continuations(model, toks[i:i + bsz].cuda(), ctx[i:i + bsz].cuda(), total[i:i + bsz].cuda())
            e1.record()
            barrier()
            ms_score = max_over_ranks(e0.elapsed_time(e1), rt)
            prompts = toks[:a.decode_batch, :64].cuda()
            greedy_decode(model, prompts, 4)
            barrier()
            e0.record()
            out = greedy_decode(model, prompts, a.new_tokens)
            e1.record()
            barrier()
            ms_dec = max_over_ranks(e0.elapsed_time(e1), rt)
        _lib.check_error_word()
        if rt.rank == 0:
            print(json.dumps({"what": "infer", "n_gpus": rt.world,
                              "scoring_tokens_per_s": rt.world * n * 2048 / (ms_score / 1e3), "scoring_requests": rt.world * n,
                              "decode_tokens_per_s": rt.world * a.decode_batch * a.new_tokens / (ms_dec / 1e3),
                              "decode_batch": a.decode_batch, "new_tokens": a.new_tokens, "ms_score": ms_score, "ms_decode": ms_dec,
                              "config": {"model": f"dense {a.depth}Lx1280 replica per rank", "kv_cache": True,
                                         "scoring_path": "native kernels", "decode_path": "native kernels in a CUDA graph, KV cache"},
                              "sample": out[0, -4:].tolist(), "mean_score": float(s.mean())}), flush=True)
    if rt.ddp:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
