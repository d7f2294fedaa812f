"""Training entry point: ``torchrun --standalone --nproc_per_node=N train.py [flags]`` (or plain ``python train.py``).

Flow (reference ``main()``: round2/source/train.py:21339-23503): flags and environment recipe -> runtime init -> model,
optimizer, tables -> synthetic loader with a prefetch worker -> step loop with schedules, collective step control, the
asynchronous step boundary, predictive stop rule, rescue copy, log line every 10 steps -> final checkpoint
``{"model_state","model_config","meta"}`` -> causality check and bits-per-byte evaluation -> summary block.

``--compile-only`` runs one synthetic zero-token step through every kernel and optimizer path and exits (reference:
round2/source/train.py:21910-21996).
"""
from __future__ import annotations

import argparse
import json
import math
import os
import sys
import time

import torch

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

from them_bones_b200 import config as C  # noqa: E402
from them_bones_b200 import ops  # noqa: E402
from them_bones_b200.data.synth import Prefetcher, SynthLoader  # noqa: E402
from them_bones_b200.runtime import StepTimer, cleanup_runtime, init_runtime, print0  # noqa: E402
from them_bones_b200.trainer import Trainer  # noqa: E402
from them_bones_b200.utils import ckpt as CK  # noqa: E402
from them_bones_b200.utils.control import AsyncBoundary, StepControl, StopRule  # noqa: E402
from them_bones_b200.utils.ema import EmaLawa  # noqa: E402
from them_bones_b200.utils.evalbpb import causality_check, evaluate_bpb  # noqa: E402
from them_bones_b200.utils.memprobe import MemPhase, MicroBarrier, memory_line  # noqa: E402
from them_bones_b200.utils.shed import ShedProbe  # noqa: E402


def parse_args(argv=None):
    e = os.environ.get
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--recipe", default=e("BONES_RECIPE", ""), help="KEY=VALUE environment recipe file")
    ap.add_argument("--depth", type=int, default=int(e("BONES_DEPTH", 20)))
    ap.add_argument("--n-embd", type=int, default=int(e("BONES_N_EMBD", 1280)))
    ap.add_argument("--n-head", type=int, default=int(e("BONES_N_HEAD", 10)))
    ap.add_argument("--head-dim", type=int, default=int(e("BONES_HEAD_DIM", 0)))
    ap.add_argument("--seq-len", type=int, default=int(e("BONES_SEQ_LEN", 2048)))
    ap.add_argument("--vocab", type=int, default=int(e("BONES_VOCAB", 65536)))
    ap.add_argument("--steps", type=int, default=int(e("BONES_STEPS", 0)), help="optimizer steps (0: run on the clock)")
    ap.add_argument("--budget-seconds", type=float, default=float(e("BONES_BUDGET_SECONDS", 0)))
    ap.add_argument("--doc-len", default=e("BONES_DOC_LEN", "128,2048"))
    ap.add_argument("--out", default=e("BONES_OUT", "final.pt"))
    ap.add_argument("--no-save", action="store_true")
    ap.add_argument("--resume", default=e("BONES_RESUME", ""), help="checkpoint to continue from (weights, tables and, "
                    "when <path>.opt.rank<r> files exist, the optimizer state; same world size)")
    ap.add_argument("--eval-tokens", type=int, default=int(e("BONES_EVAL_TOKENS", 0)))
    ap.add_argument("--compile-only", action="store_true")
    ap.add_argument("--device", default=e("BONES_DEVICE", ""))
    ap.add_argument("--jsonl", default=e("BONES_JSONL", ""), help="machine-readable step log")
    return ap.parse_args(argv)


def main(argv=None):
    args = parse_args(argv)
    if args.recipe:
        C.load_recipe(args.recipe)
        args = parse_args(argv)                              # recipe values are defaults for the geometry flags
    hyper = C.Hyper.from_env()
    sw = C.switches(refresh=True)
    rt = init_runtime(args.device or None, seed=hyper.seed)
    print0(f"device {rt.device} world {rt.world} kernels {'ref' if ops.reference_path() else 'native'}")
    if sw["SELFCHECK"] and rt.device_type == "cuda" and not ops.reference_path():
        from them_bones_b200.ops.selfcheck import run as selfcheck
        worst = max(selfcheck(rt.device).values())
        print0(f"self-check: native kernels agree with the PyTorch path (worst relative error {worst:.2e})")
    cfg = C.build_config(args.depth, args.n_embd, args.n_head, args.seq_len, args.vocab, head_dim=args.head_dim,
                         hyper=hyper)
    print0("model_config " + json.dumps(C.model_config_dict(cfg)))
    init_state, resumed_steps = None, 0
    if args.resume:
        ck = torch.load(args.resume, map_location="cpu", weights_only=True, mmap=True)
        if ck["model_config"] != C.model_config_dict(cfg):
            raise ValueError("--resume: the checkpoint's model_config differs from this run's")
        init_state, resumed_steps = ck["model_state"], int(ck.get("meta", {}).get("steps", 0))
    tr = Trainer(cfg, hyper, rt, horizon_steps=args.steps, budget_seconds=args.budget_seconds, init_state=init_state)
    if args.resume:
        opt_file = CK.opt_state_path(args.resume, rt.rank)
        if os.path.exists(opt_file) and hasattr(tr.optimizer, "load_unit_state_dict"):
            tr.optimizer.load_unit_state_dict(torch.load(opt_file, map_location="cpu", weights_only=True))
        tr.step_index = resumed_steps               # step-driven schedules continue where the checkpoint stopped
        print0(f"resumed from {args.resume} (checkpoint step {resumed_steps}, optimizer state "
               f"{'loaded' if os.path.exists(opt_file) else 'fresh'})")
    if sw["ANSWER_PHASE"] > 0:
        tr.model.answer_weight = sw["ANSWER_WEIGHT"]     # marked targets are unmarked and weighted inside the forward
    print0(tr.describe())
    n_params = tr.model.num_scaling_params()
    print0(f"parameters {n_params:,}; flops/token {tr.flops_per_token:.4e}")
    lo, hi = (int(v) for v in args.doc_len.split(","))
    from them_bones_b200.data.select import DocRule
    rule = DocRule.parse(sw["DATA_RULE"], cfg.vocab_size, cfg.bos_id)
    from them_bones_b200.data.streams import Streams
    streams = Streams.parse(sw["DATA_STREAMS"], vocab=cfg.vocab_size, seq_len=cfg.sequence_len, bos_id=cfg.bos_id, rank=rt.rank,
                            world=rt.world, seed=hyper.seed)
    loader = SynthLoader(cfg.vocab_size, cfg.sequence_len, tr.local_windows, rank=rt.rank, seed=hyper.seed,
                         doc_len=(lo, min(hi, cfg.sequence_len * 4)), bos_id=cfg.bos_id, pin=rt.device_type == "cuda",
                         rule=rule, streams=streams)
    if args.compile_only:
        x = torch.zeros(tr.local_windows, cfg.sequence_len, dtype=torch.int32)
        y = torch.zeros(tr.local_windows, cfg.sequence_len, dtype=torch.int64)
        loss = tr.train_step(x if rt.device_type == "cuda" else x.long(), y)
        print0(f"compile-only step ok, loss {float(loss):.4f}; native op counts {dict(ops.COUNTS)}")
        cleanup_runtime()
        return 0
    fetch = (lambda: loader.next_step())
    prefetch = Prefetcher(fetch) if sw["PREFETCH"] else None
    control = StepControl(rt, hyper.bad_loss)
    stop_rule = StopRule(args.budget_seconds, reserve_s=0.02 * args.budget_seconds)
    boundary = AsyncBoundary(rt.device, hyper.sync_every) if sw["BOUNDARY_ASYNC"] else None
    rescue = CK.RescueCopy(hyper.rescue_from, hyper.rescue_every)
    bg_save = CK.BackgroundSave()
    memphase = MemPhase(rt.device, sw["MEM_PHASE"])
    ema = EmaLawa(tr.model.parameters(), 1.0 - sw["EMA"], 10) if sw["EMA"] > 0 else None
    shed = ShedProbe(rt, tr.grad_accum) if sw["SHED"] else None
    micro_barrier = MicroBarrier(rt.device) if sw["MICRO_BARRIER"] else None  # noqa: F841 (ticks inside Trainer hooks)
    timer = StepTimer(rt)
    jsonl = open(args.jsonl, "a") if (args.jsonl and rt.is_master) else None
    tokens_per_step = tr.total_batch
    ema_loss, dts, step, bad = 0.0, [], 0, False
    t_train0 = time.time()
    if prefetch:
        prefetch.start()
    ramp_until = sw["SEQ_RAMP"]
    while True:
        if args.steps and step >= args.steps:
            break
        memphase.begin(step)
        if ramp_until > 0:
            want = cfg.sequence_len // 2 if tr.progress() < ramp_until else cfg.sequence_len
            if loader.seq_len != want:
                loader.set_seq_len(want)
                print0(f"step {step}: window length -> {want}")
        if rule is not None:
            rule.phase = tr.progress()
        if streams is not None:
            streams.set_phase(tr.progress())
        if sw["ANSWER_PHASE"] > 0 and loader.mark_tail == 0.0 and tr.progress() >= 1.0 - sw["ANSWER_PHASE"]:
            loader.mark_tail = sw["ANSWER_TAIL"]         # rows fetched from here on carry answer-span marks
            print0(f"step {step}: answer phase on (tail {sw['ANSWER_TAIL']}, weight {sw['ANSWER_WEIGHT']})")
        x, y = prefetch.finish() if prefetch else fetch()
        if prefetch:
            prefetch.start()
        if rt.device_type == "cpu":
            x = x.long()
        if x.shape[1] != cfg.sequence_len:                    # ramp: same tokens, shorter windows
            tr.grad_accum_saved = tr.grad_accum
        timer.start()
        t_host0 = time.perf_counter()
        micro = None
        if shed is not None and step > hyper.startup_steps_excluded:
            micro, _ = shed.counts[rt.rank], None
        loss = tr.train_step(x, y, micro_steps=micro)
        memphase.mark("step")
        loss_value = None
        sync_now = boundary is None or boundary.must_sync(step) or bool(args.steps and step == args.steps - 1)
        if boundary is not None:
            prev = boundary.collect() if boundary.pending is not None else None
            boundary.submit(step, loss)
            if sync_now:
                prev = boundary.collect()
            if prev is not None:
                loss_value = prev[1]
        if sync_now:
            dt = timer.stop() / 1e3
            if boundary is None:
                loss_value = float(loss)
            # a forced synchronous boundary is where latent device errors surface: a bounded wait that ran out inside a
            # kernel (peer barrier, mbarrier) left its code in the error word, and the fused optimizer kernels counted
            # the steps whose reduced gradient held a non-finite value
            tr.check_device_health()
        else:
            # asynchronous boundary: the host runs at most a queue's depth ahead, so in steady state the host time per
            # loop iteration equals the device time per step
            dt = time.perf_counter() - t_host0
        if shed is not None:
            shed.update(dt * 1e3)
        if step >= hyper.startup_steps_excluded or (args.steps and args.steps <= hyper.startup_steps_excluded and step > 0):
            dts.append(dt)              # runs shorter than the start-up exclusion report all but their first step
            stop_rule.observe(dt)
        if step == hyper.startup_steps_excluded:
            t_train0 = time.time()
            tr.t_start = t_train0
        elapsed = time.time() - t_train0
        want_stop = stop_rule.should_stop(elapsed)
        bad, stop, clock_ms = control.decide(loss_value, want_stop, elapsed * 1e3)
        if step >= hyper.startup_steps_excluded:
            tr.set_agreed_clock(clock_ms / 1e3)      # every clock-driven decision below and in the next step uses it
        if loss_value is not None:
            ema_loss = 0.9 * ema_loss + 0.1 * loss_value
        if step % hyper.log_every == 0 and loss_value is not None:
            deb = ema_loss / (1 - 0.9 ** (step + 1))
            tps = tokens_per_step / dt if dt > 0 else 0.0
            print0(f"step {step:6d} | loss {deb:.4f} | lrm {tr.sched['lrm']:.3f} | dt {dt * 1e3:8.1f} ms | "
                   f"tok/s {tps:12,.0f} | clock {elapsed:7.1f}s")
            if jsonl:
                jsonl.write(json.dumps(dict(step=step, loss=loss_value, dt_ms=dt * 1e3, tok_s=tps,
                                            lrm=tr.sched["lrm"])) + "\n")
                jsonl.flush()
            if tr.last_moe_stats is not None and step % (10 * hyper.log_every) == 0:
                st = tr.last_moe_stats.float().mean(0).tolist()
                print0(f"   moe: kept {st[0]:.3f} balance {st[1]:.3f} z {st[2]:.3f} max share {max(st[3:]):.3f}")
        if sw["MEM_PRINT"] and step == 10:
            print0(memory_line(rt.device))
        if bad:
            print0(f"step {step}: bad loss {loss_value}; leaving the loop")
            if rescue.state is not None:
                CK.save_checkpoint(args.out + ".rescue", tr.model, dict(step=rescue.step, rescue=True), rank=rt.rank,
                                   state=rescue.state)
            else:
                cleanup_runtime()
                raise RuntimeError("loss went bad before a rescue copy existed")
            break
        if ema is not None:
            ema.update(step, tr.progress())
        rescue.maybe_refresh(step, tr.progress(), tr.model, tr.optimizer)
        if sw["SAVE_EVERY"] > 0 and step > 0 and step % sw["SAVE_EVERY"] == 0 and not args.no_save:
            payload = CK.build_payload(tr.model, dict(steps=step, periodic=True), tr.optimizer, tr.tables)
            if rt.is_master:
                bg_save.submit(args.out + ".periodic", payload)
        step += 1
        if stop:
            print0(f"step {step}: stop rule fired at {elapsed:.1f}s")
            break
    if memphase.rows:
        print0("mem-phase: " + memphase.report())
    averaged = ema is not None and ema.avg is not None
    if averaged:
        ema.swap_in()
    total_s = time.time() - t_train0
    meta = dict(steps=step, tokens=step * tokens_per_step, seconds=total_s, switches=sw, world=rt.world,
                median_dt=sorted(dts)[len(dts) // 2] if dts else None, bad=bad, native_ops=dict(ops.COUNTS),
                save_opt_state=sw["SAVE_OPT_STATE"])
    bg_save.wait()
    tr.check_device_health()
    meta["bad_steps"] = tr.bad_steps
    if not args.no_save:
        CK.check_declared_length(tr.model, loader.seq_len)
        # after the tail average was swapped in, the in-memory replicas are the model (the owners' fp32 masters still
        # hold the un-averaged weights), so the file is written from the replicas and equals what is evaluated below
        CK.save_checkpoint(args.out, tr.model, meta, optimizer=None if averaged else tr.optimizer, tables=tr.tables,
                           rank=rt.rank)
        if sw["SAVE_OPT_STATE"]:
            CK.save_optimizer_state(args.out, tr.optimizer, rt.rank)
        print0(f"saved {args.out}")
    result = {}
    if args.eval_tokens:
        cc = causality_check(tr.model, cfg.vocab_size, 2, cfg.sequence_len, rt.device)
        ev = evaluate_bpb(tr.model, cfg.vocab_size, tr.device_batch, cfg.sequence_len, rt.device,
                          max_tokens=args.eval_tokens, bos_id=cfg.bos_id)
        result.update(causality=cc, **ev)
        print0(f"causality passed={cc['passed']} max_abs_diff={cc['max_abs_diff']:.3e}; val_bpb {ev['val_bpb']:.4f}")
        if sw["EVAL_SPLIT"]:
            # per-class held-out loss; the contexts of one training-stream row stand for "text the run has seen"
            from them_bones_b200.utils.evalsplit import ContextSet, evaluate_split
            seen = ContextSet(ctx=8)
            seen.add(loader.rows.next_row())
            split = evaluate_split(tr.model, cfg.vocab_size, tr.device_batch, cfg.sequence_len, rt.device,
                                   max_tokens=args.eval_tokens, bos_id=cfg.bos_id, contexts=seen, rank=rt.rank)
            result.update(eval_split=split)
            print0("eval_split " + json.dumps({k: round(v["bpb"], 4) for k, v in split.items()}))
    med = meta["median_dt"]
    print0("---")
    print0(f"steps {step} tokens {meta['tokens']:,} seconds {total_s:.1f} median_dt "
           f"{(med or 0) * 1e3:.1f} ms tok/s {(tokens_per_step / med) if med else 0:,.0f} final_loss "
           f"{ema_loss / max(1e-9, 1 - 0.9 ** max(step, 1)):.4f}")
    print0(f"native op counts: {dict(ops.COUNTS)}")
    if rule is not None:
        print0(rule.line())
    for ln in (streams.lines() if streams is not None else []):
        print0(ln)
    if sw["MEM_PRINT"]:
        print0(memory_line(rt.device))
    cleanup_runtime()
    return 0


if __name__ == "__main__":
    sys.exit(main())
