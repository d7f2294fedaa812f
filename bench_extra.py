"""Secondary benchmarks (the headline benchmark is ``bench.py``): MoE training, MoE + hashed tables, inference.

    python bench_extra.py --what moe    [--gpus N under torch.distributed.run] --steps 2 --warmup 2
    python bench_extra.py --what full   --table-rows 4194304          (MoE + bigram/trigram tables)
    python bench_extra.py --what os1    --os1-rows 16777216            (dense decoder + output-side table)
    python bench_extra.py --what infer  --requests 4096 --decode-batch 64 --new-tokens 128 --table-rows 1048576

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
    ap.add_argument("--mlp", default=os.environ.get("BONES_MLP", "mxfp8"), help="MLP / expert GEMM precision: mxfp8 | bf16")
    ap.add_argument("--ckpt-dir", default="", help="infer: where the synthetic checkpoint is written (default: the temp dir)")
    a = ap.parse_args()

    import torch
    import torch.distributed as dist

    from them_bones_b200 import ops
    from them_bones_b200.config import GPTConfig, Hyper, moe_capacity_for
    from them_bones_b200.data.synth import SynthLoader
    from them_bones_b200.ops import _lib
    from them_bones_b200.runtime import init_runtime, max_over_ranks

    rt = init_runtime("cuda")
    kw = dict(sequence_len=2048, vocab_size=65536, n_layer=a.depth, n_head=10, n_embd=1280, head_dim=128, doc_mask=True,
              mlp_precision=a.mlp)
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
                                         "global_batch": tr.total_batch, "experts_per_gpu": 16 // rt.world, "mlp_precision": a.mlp,
                                         "fused_comm": tr.comm is not None},
                              "os1_stats": tr.os1.stats if tr.os1 is not None else None,
                              "native_ops": dict(ops.COUNTS), "moe_stats": (tr.last_moe_stats.float().mean(0)[:3].tolist()
                                                                            if tr.last_moe_stats is not None else None)}), flush=True)
    else:
        # Inference as configured: a random-init checkpoint of the MoE + tables model in the reference layout is written
        # once, loaded back through the public ``inference.load_for_eval`` and served sharded over the ranks (experts by
        # the fused dispatch, table rows by peer gathers); every rank scores its share of the requests and decodes its own
        # batch, in lockstep.
        import tempfile
        import time

        import inference
        from them_bones_b200.models.gpt import GPT
        from them_bones_b200.models.tables import HashedTables
        from them_bones_b200.utils import ckpt as CK
        cfg_i = GPTConfig(**{**kw, "table_orders": (2, 3), "table_rows": a.table_rows})
        path = os.path.join(a.ckpt_dir or tempfile.gettempdir(), f"bones_infer_{a.depth}_{a.table_rows}.pt")
        t0 = time.time()
        if rt.rank == 0 and not os.path.exists(path):
            torch.manual_seed(0)
            full = GPT(cfg_i)
            full.init_weights()
            with torch.no_grad():
                for blk in full.transformer.h:            # non-zero output projections: a random model that does something
                    blk.attn.c_proj.weight.normal_(0, 0.02)
                    (blk.mlp.w_proj if hasattr(blk.mlp, "w_proj") else blk.mlp.c_proj.weight).normal_(0, 0.02)
                full.lm_head.weight.normal_(0, 0.02)
            tabs = HashedTables(cfg_i.table_orders, cfg_i.table_rows, cfg_i.n_embd, dtype=torch.bfloat16)
            for sh in tabs.shards:
                sh.normal_(0, 0.1)
            CK.save_checkpoint(path, full.to(torch.bfloat16), dict(steps=0, synthetic=True), tables=tabs)
            del full, tabs
        barrier()
        t_ckpt = time.time() - t0
        t0 = time.time()
        wrapper = inference.load_for_eval(path, rt.device, rt=rt if rt.world > 1 else None)
        model = wrapper.model
        barrier()
        t_load = time.time() - t0
        g = torch.Generator().manual_seed(rt.rank)
        n, bsz = max(a.requests // rt.world, 8), 8
        toks = torch.randint(1, 65536, (n, 2048), generator=g)
        toks[:, 0] = 0
        total = torch.randint(512, 2049, (n,), generator=g)
        cont = torch.randint(1, 65, (n,), generator=g)
        ctx = total - cont
        with torch.no_grad():
            wrapper.score(toks[:bsz].cuda(), ctx[:bsz].cuda(), total[:bsz].cuda())
            barrier()
            e0.record()
            for i in range(0, n, bsz):
                s = wrapper.score(toks[i:i + bsz].cuda(), ctx[i:i + bsz].cuda(), total[i:i + bsz].cuda())
            e1.record()
            barrier()
            ms_score = max_over_ranks(e0.elapsed_time(e1), rt)
            prompts = toks[:a.decode_batch, :64].cuda()
            wrapper.generate(prompts, 4)
            barrier()
            e0.record()
            out = wrapper.generate(prompts, a.new_tokens)
            e1.record()
            barrier()
            ms_dec = max_over_ranks(e0.elapsed_time(e1), rt)
        _lib.check_error_word()
        if rt.rank == 0:
            print(json.dumps({"what": "infer", "n_gpus": rt.world,
                              "scoring_tokens_per_s": rt.world * n * 2048 / (ms_score / 1e3), "scoring_requests": rt.world * n,
                              "decode_tokens_per_s": rt.world * a.decode_batch * a.new_tokens / (ms_dec / 1e3),
                              "decode_batch": a.decode_batch, "new_tokens": a.new_tokens, "ms_score": ms_score, "ms_decode": ms_dec,
                              "config": {"model": f"moe 16e top-2 {a.depth}Lx1280 + bigram/trigram tables {a.table_rows} rows x 1280",
                                         "checkpoint": "reference layout, loaded by inference.load_for_eval",
                                         "sharded": rt.world > 1, "experts_per_gpu": 16 // rt.world,
                                         "peer_memory": getattr(model, "comm", None) is not None,
                                         "decode_path": "native kernels in a CUDA graph, KV cache",
                                         "checkpoint_write_s": round(t_ckpt, 1), "load_s": round(t_load, 1)},
                              "native_ops": dict(ops.COUNTS), "sample": out[0, -4:].tolist(), "mean_score": float(s.mean())}),
                  flush=True)
    if rt.ddp:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
