"""Headline benchmark: training tokens/s of the round-1 dense decoder (20 layers x 1280, 10 heads x 128, ReLU^2 MLP
1280->5120->1280, vocab 65536, sequence 2048, document-reset causal attention, Muon+AdamW, global batch 524288 tokens)
on N GPUs of one node, synthetic Zipf(1.1) tokens and random-init weights.

    python bench.py --gpus 1 --steps K --warmup W
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P \
        bench.py --gpus N --steps K --warmup W

Prints one JSON line on rank 0.  ``value`` is the whole-job tokens/s timed on the device (CUDA events, max over ranks)
with the step's inputs already resident; ``e2e.value`` times the same K steps through the public ``Trainer.train_step``
call including the pinned host-to-device copy of every step's tokens and a device-to-host read of every step's loss.
Global batch is fixed as N grows (strong scaling).  ``--impl reference`` runs the reference arm.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)

PUBLISHED_TOK_S = 340000.0      # reference round-1 throughput on one Trainium2 chip (round1/README.md:24)


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi (read-only).  The process is started before the warm-up,
    because nvidia-smi needs about a second before its first line; only lines read between ``mark_begin()`` and
    ``stop()`` -- the timed region -- are used."""

    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu_index, self.proc, self.lines, self.t_begin = gpu_index, None, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                                          "-lms", "100", "-i", str(self.gpu_index)], stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._pump, daemon=True).start()
        except OSError:
            self.proc = None

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append((time.time(), line.strip()))

    def mark_begin(self):
        self.t_begin = time.time()

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, smax, power, reasons = [], [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        t_end = time.time()
        for ts, ln in self.lines:
            if self.t_begin is not None and not (self.t_begin <= ts <= t_end):
                continue
            parts = [p.strip() for p in ln.split(",")]
            if len(parts) < 9:
                continue
            try:
                sm.append(float(parts[1])); smax.append(float(parts[2])); power.append(float(parts[3]))
            except ValueError:
                continue
            for name, val in zip(names, parts[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(smax) if smax else None,
                "power_w_max": max(power) if power else None, "samples": len(sm), "reasons": sorted(reasons)}


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference", "torch"])
    ap.add_argument("--device-batch", type=int, default=int(os.environ.get("BONES_DEVICE_BATCH", 64)),
                    help="sequences per micro-step per GPU (clamped to the rank's share of the global batch)")
    ap.add_argument("--total-batch", type=int, default=524288)
    ap.add_argument("--depth", type=int, default=20)
    ap.add_argument("--mlp", default=os.environ.get("BONES_MLP", "mxfp8"),
                    help="MLP GEMM precision: mxfp8 (block-scaled, the benchmark configuration) or bf16")
    ap.add_argument("--attn-proj", default=os.environ.get("BONES_ATTN_PROJ", "bf16"))
    return ap.parse_args()


def run_ours(args, torch_path: bool = False):
    import torch
    import torch.distributed as dist

    from them_bones_b200 import ops
    from them_bones_b200.config import GPTConfig, Hyper
    from them_bones_b200.data.synth import SynthLoader
    from them_bones_b200.ops import _lib
    from them_bones_b200.runtime import init_runtime, max_over_ranks

    if torch_path:
        ops.set_reference_path(True)
    rt = init_runtime("cuda")
    if rt.world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE is {rt.world}: launch with torch.distributed.run")
    cfg = GPTConfig(sequence_len=2048, vocab_size=65536, n_layer=args.depth, n_head=10, n_embd=1280, head_dim=128,
                    doc_mask=True, mlp_precision=args.mlp, attn_proj_precision=args.attn_proj)
    hyper = Hyper()
    # the global batch is fixed, so with more GPUs a rank's share shrinks below the preferred micro-batch
    from them_bones_b200.config import micro_batch_for
    pref = args.device_batch if not torch_path else min(args.device_batch, 32)       # the PyTorch bodies hold whole logits
    hyper.total_batch, hyper.device_batch = args.total_batch, micro_batch_for(args.total_batch, rt.world, pref, 2048)
    from them_bones_b200.trainer import Trainer
    tr = Trainer(cfg, hyper, rt, horizon_steps=10000)
    # one stream for the whole job, rank r keeping windows r, r + W, ...: every rank count sees the same global batches,
    # so `final_loss` is comparable across N
    loader = SynthLoader(cfg.vocab_size, cfg.sequence_len, tr.local_windows, rank=rt.rank, seed=hyper.seed,
                         doc_len=(128, 2048), bos_id=cfg.bos_id, pin=True, shard_of=rt.world)
    n_batches = max(2, min(4, args.steps))
    host = [loader.next_step() for _ in range(n_batches)]         # pinned host windows, larger than L2 per step
    dev = [(x.to(rt.device), y.to(rt.device)) for x, y in host[:2]]

    def barrier():
        if rt.ddp:
            dist.barrier()
        torch.cuda.synchronize()

    sampler = ClockSampler(rt.local_rank)
    sampler.start()
    for i in range(args.warmup):
        tr.train_step(*dev[i % 2])
    barrier()
    _lib.check_error_word() if not torch_path else None
    # ---- device-timed region: inputs resident, CUDA events on the launching stream ----
    launches0 = _lib.LAUNCHES[0]
    counts0 = dict(ops.COUNTS)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    sampler.mark_begin()
    tr.time_optimizer = True
    e0.record()
    for i in range(args.steps):
        loss = tr.train_step(*dev[i % 2])
    e1.record()
    barrier()
    tr.time_optimizer = False
    opt_ms = max_over_ranks(sum(a.elapsed_time(b) for a, b in tr.optimizer_events) / max(1, len(tr.optimizer_events)), rt)
    clocks = sampler.stop()
    ms = max_over_ranks(e0.elapsed_time(e1), rt)
    launches = _lib.LAUNCHES[0] - launches0
    tokens = args.steps * tr.total_batch
    value = tokens / (ms / 1e3)
    # ---- end-to-end region: pinned host -> device copy of each step's tokens, device -> host loss read per step ----
    pinned_loss = torch.zeros(1, dtype=torch.float32).pin_memory()
    h2d = host[0][0].numel() * host[0][0].element_size() + host[0][1].numel() * host[0][1].element_size()
    barrier()
    t0 = time.perf_counter()
    e0.record()
    last = 0.0
    for i in range(args.steps):
        x, y = host[i % n_batches]
        loss = tr.train_step(x, y)
        pinned_loss.copy_(loss.reshape(1).float(), non_blocking=False)
        last = float(pinned_loss[0])
    e1.record()
    barrier()
    wall_ms = (time.perf_counter() - t0) * 1e3
    if rt.ddp:        # outside the timed region: the last step's loss as the mean over all ranks' windows
        t = torch.tensor([last], device=rt.device)
        dist.all_reduce(t)
        last = float(t[0]) / rt.world
    ms_e2e = max_over_ranks(max(e0.elapsed_time(e1), wall_ms), rt)
    e2e_value = tokens / (ms_e2e / 1e3)
    if not torch_path:
        _lib.check_error_word()
    # steps whose reduced gradient held a non-finite value (the fused optimizer zeroes those entries and counts the step)
    bad_steps = tr.optimizer.count_bad_steps() if hasattr(tr.optimizer, "count_bad_steps") else 0
    if rt.rank == 0:
        out = {
            "metric": "train tokens/sec (device-timed, max over ranks)", "value": value, "unit": "tokens/s",
            "n_gpus": rt.world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms / args.steps,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": value / PUBLISHED_TOK_S, "dtype": "bf16",
            "data": "synthetic Zipf(1.1) tokens, documents 128-2048, random-init weights",
            "impl": "torch" if torch_path else "ours",
            "config": {"model": "round1-dense 20Lx1280 10hx128 relu2-mlp x4 vocab65536" if args.depth == 20 else
                       f"dense {args.depth}Lx1280", "global_batch": tr.total_batch, "seq_len": 2048,
                       "parallelism": f"dp{rt.world}", "device_batch": tr.device_batch, "grad_accum": tr.grad_accum,
                       "mlp_precision": args.mlp, "attn_proj_precision": args.attn_proj, "optimizer": "Muon+AdamW (sharded)",
                       "l2": "inputs and activations per step exceed L2 (126 MB); two alternating batches"},
            "clocks": clocks,
            "e2e": {"value": e2e_value, "unit": "tokens/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": 4,
                    "ms_per_step": ms_e2e / args.steps, "final_loss": last},
            "gpu_launches": int(launches),
            "optimizer_ms_per_step": opt_ms,      # device time of the step-boundary optimizer chain, max over ranks
            "non_finite_steps": int(bad_steps),
            "native_ops": {k: v - counts0.get(k, 0) for k, v in ops.COUNTS.items()},
            "tflops_per_gpu": value * tr.flops_per_token / rt.world / 1e12,
            "peak_mem_gb": torch.cuda.max_memory_allocated() / 2 ** 30,
        }
        print(json.dumps(out), flush=True)
    if rt.ddp:
        dist.barrier()
        dist.destroy_process_group()


def main():
    args = parse()
    if args.impl == "reference":
        from baseline import reference_arm
        return reference_arm.main(args)
    run_ours(args, torch_path=args.impl == "torch")


if __name__ == "__main__":
    main()
