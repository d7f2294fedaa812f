"""CPU tests: configuration, synthetic data, schedules, optimizer math, MXFP8 emulation, control utilities."""
import math
import os

import numpy as np
import pytest
import torch

from them_bones_b200 import config as C
from them_bones_b200.data import synth
from them_bones_b200.optim import schedules as S
from them_bones_b200.ref import functional as RF


def test_env_parsing_and_refusals(monkeypatch):
    monkeypatch.setenv("BONES_UNET", "1")
    monkeypatch.setenv("BONES_MLP", "mxfp8")
    s = C.switches(refresh=True)
    assert s["UNET"] is True and s["MLP"] == "mxfp8"
    monkeypatch.setenv("BONES_UNET", "yes")
    with pytest.raises(ValueError):
        C.switches(refresh=True)
    monkeypatch.setenv("BONES_UNET", "0")
    monkeypatch.setenv("BONES_SHED", "1")
    monkeypatch.setenv("BONES_MOE", "1")
    with pytest.raises(ValueError):
        C.switches(refresh=True)
    monkeypatch.delenv("BONES_SHED")
    monkeypatch.delenv("BONES_MOE")
    monkeypatch.delenv("BONES_MLP")
    C.switches(refresh=True)


def test_recipe_file_and_config_roundtrip(tmp_path, monkeypatch):
    p = tmp_path / "r.env"
    p.write_text("# comment\nexport BONES_DOC_MASK=1\nBONES_ATTN_WINDOW=256  # trailing\n")
    monkeypatch.delenv("BONES_DOC_MASK", raising=False)
    monkeypatch.delenv("BONES_ATTN_WINDOW", raising=False)
    got = C.load_recipe(str(p))
    assert got == {"BONES_DOC_MASK": "1", "BONES_ATTN_WINDOW": "256"}
    C.switches(refresh=True)
    cfg = C.build_config(8, 256, 2, 512, 8192, head_dim=128)
    assert cfg.doc_mask and cfg.attn_window == 256 and cfg.attn_long == (3, 7)
    d = C.model_config_dict(cfg)
    assert "unet" not in d and d["attn_window"] == 256
    assert C.GPTConfig(**d) == cfg
    for k in got:
        monkeypatch.delenv(k)
    C.switches(refresh=True)


def test_moe_capacity_and_layer_parsing():
    assert C.moe_capacity_for(1.25, 2048, 1, 64) == 40
    assert C.moe_capacity_for(1.25, 2048, 2, 16) == 320
    assert C.parse_layers("2:", 6) == (2, 3, 4, 5)
    assert C.parse_layers("1,3", 6) == (1, 3)
    with pytest.raises(ValueError):
        C.parse_layers("9", 6)


def test_zipf_stream_is_deterministic_and_skewed():
    a = synth.ZipfDocs(8192, 1.1, (16, 64), seed=3).tokens(20000)
    b = synth.ZipfDocs(8192, 1.1, (16, 64), seed=3).tokens(20000)
    assert (a == b).all() and a.min() >= 1 and a.max() < 8192
    counts = np.bincount(a, minlength=8192)
    assert counts[1] > counts[10] > counts[1000]
    ratio = counts[1] / max(1, counts[2])
    assert 1.5 < ratio < 3.0                      # 2**1.1 = 2.14


def test_packed_rows_windows_and_bos_mask():
    ld = synth.SynthLoader(8192, 256, 8, seed=1, doc_len=(64, 512))
    x, y = ld.next_step()
    assert x.shape == (8, 256) and y.shape == (8, 256) and x.dtype == torch.int32 and y.dtype == torch.int64
    flat_x, flat_y = x.reshape(-1), y.reshape(-1)
    assert flat_x[0] == 0                                                  # a row starts with a document
    nxt = flat_x[1:].long()
    assert ((flat_y[:-1] == nxt) | ((nxt == 0) & (flat_y[:-1] == -1))).all()  # shifted by one, BOS targets masked
    assert (flat_y != 0).all()
    ld.set_seq_len(128)
    x2, _ = ld.next_step()
    assert x2.shape == (16, 128)


def test_prefetcher_surfaces_worker_exception():
    def boom():
        raise RuntimeError("worker died")
    p = synth.Prefetcher(boom)
    p.start()
    with pytest.raises(RuntimeError, match="worker died"):
        p.finish()


def test_schedules():
    assert S.lr_multiplier(0.0, 0, 40, 0.85, 0.01) == pytest.approx(1 / 40)
    assert S.lr_multiplier(0.1, 100, 40, 0.85, 0.01) == 1.0
    assert S.lr_multiplier(1.0, 1000, 40, 0.85, 0.01) == pytest.approx(0.01)
    mid = S.lr_multiplier(0.575, 1000, 40, 0.85, 0.01)
    assert 0.01 < mid < 1.0
    assert S.muon_momentum(0, 0.0, 0.65) == pytest.approx(0.85)
    assert S.muon_momentum(300, 0.1, 0.65) == pytest.approx(0.97)
    assert S.muon_momentum(5000, 1.0, 0.65) == pytest.approx(0.90)
    assert S.grad_accum_for_step(0.1, 8, 0.3) == 4 and S.grad_accum_for_step(0.5, 8, 0.3) == 8


def test_newton_schulz_orthogonalises():
    torch.manual_seed(0)
    for shape in ((2, 64, 32), (2, 32, 64)):
        x = torch.randn(*shape)
        x = x / (x.norm(dim=(-2, -1), keepdim=True) * 1.01 + 1e-6)
        y = RF.newton_schulz(x, 5)
        s = torch.linalg.svdvals(y)
        assert s.max() < 1.3 and s.min() > 0.5


def test_muon_update_matches_manual_reference():
    torch.manual_seed(1)
    n, r, c = 3, 48, 32
    g = torch.randn(n, r, c)
    w0 = torch.randn(n, r, c)
    w, mom, sec = w0.clone(), torch.zeros(n, r, c), torch.zeros(n, r, 1)
    RF.muon_update(g.clone(), w, mom, sec, momentum=0.95, beta2=0.9, lr=0.02, wd=0.05)
    # manual restatement of the same formulae
    m = 0.05 * g
    gg = g + 0.95 * (m - g)
    x = gg / (gg.norm(dim=(-2, -1), keepdim=True) * 1.01 + 1e-6)
    x = RF.newton_schulz(x, 5)
    v_mean = x.square().mean(-1, keepdim=True)
    v_norm = (v_mean.sum((-2, -1), keepdim=True) * c).sqrt()
    second = 0.1 * v_mean
    step = second.clamp_min(1e-10).rsqrt()
    v_new = ((v_mean * c) * step.square()).sum((-2, -1), keepdim=True).sqrt()
    upd = x * (step * (v_norm / v_new.clamp_min(1e-10)))
    lr = 0.02 * math.sqrt(r / c)
    ref = w0 - (lr * upd + lr * 0.05 * w0 * ((upd * w0) >= 0))
    assert torch.allclose(w, ref, atol=1e-6)
    assert torch.allclose(mom, m) and torch.allclose(sec, second)


def test_adamw_update_matches_torch():
    torch.manual_seed(2)
    p = torch.randn(10, 7)
    ref = p.clone().requires_grad_(True)
    opt = torch.optim.AdamW([ref], lr=0.01, betas=(0.8, 0.95), eps=1e-10, weight_decay=0.1)
    m, v = torch.zeros_like(p), torch.zeros_like(p)
    for step in range(1, 4):
        g = torch.randn(10, 7)
        ref.grad = g.clone()
        opt.step()
        RF.adamw_update(p, g, m, v, step=step, lr=0.01, beta1=0.8, beta2=0.95, eps=1e-10, wd=0.1)
    assert torch.allclose(p, ref.detach(), atol=1e-5)


def test_mx_quantisation_properties():
    torch.manual_seed(3)
    x = torch.randn(8, 128) * torch.logspace(-6, 3, 8)[:, None]
    q, e = RF.mx_quantize(x, -1)
    assert q.dtype == torch.float8_e4m3fn and e.shape == (8, 4) and e.dtype == torch.uint8
    back = RF.mx_dequantize(q, e, -1)
    blk = x.view(8, 4, 32)
    amax = blk.abs().amax(-1)
    scale = torch.exp2(e.float() - 127)
    assert (amax / scale <= 448.0 + 1e-3).all()                    # nothing saturates
    assert (amax / scale > 448.0 / 2 - 1e-3).all()                 # and the scale is the tightest power of two
    assert ((back - x).abs() <= blk.abs().amax(-1, keepdim=True).expand(8, 4, 32).reshape(8, 128) * 2 ** -3).all()
    z = torch.zeros(1, 32)
    qz, ez = RF.mx_quantize(z)
    assert (RF.mx_dequantize(qz, ez) == 0).all()
    col = RF.mx_qdq(x.T.contiguous(), 0)                           # quantise along the other axis
    assert torch.allclose(col.T, RF.mx_qdq(x, -1))


def test_mx_linear_close_to_fp32():
    torch.manual_seed(4)
    x, w = torch.randn(64, 256), torch.randn(96, 256) * 0.05
    rel = (RF.mx_linear(x, w) - x @ w.T).norm() / (x @ w.T).norm()
    assert rel < 0.05


def test_doc_start_and_attention_mask():
    idx = torch.tensor([[0, 5, 6, 0, 7, 8, 9, 0]])
    ds = RF.doc_start_positions(idx, 0)
    assert ds.tolist() == [[0, 0, 0, 3, 3, 3, 3, 7]]
    m = RF.attention_mask(8, "cpu", ds)[0, 0]
    assert m[2].tolist() == [True, True, True, False, False, False, False, False]
    assert m[5].tolist() == [False, False, False, True, True, True, False, False]
    band = RF.attention_mask(512, "cpu", None, window=256)[0, 0]
    assert band[511, 255] == False and band[511, 256] == True and band[300, 128] == True and band[300, 127] == False  # noqa: E712


def test_stop_rule_shed_plan_and_control():
    from them_bones_b200.runtime import Runtime
    from them_bones_b200.utils.control import AsyncBoundary, StepControl, StopRule
    from them_bones_b200.utils.shed import shed_plan
    sr = StopRule(100.0, reserve_s=5.0)
    for dt in (1.0, 1.2, 3.0):
        sr.observe(dt)
    assert not sr.should_stop(90.0) and sr.should_stop(92.5)
    counts, total = shed_plan([10, 10, 10, 20, 10, 10, 10, 10], 4)
    assert counts == [4, 4, 4, 3, 4, 4, 4, 4] and total == 31
    assert shed_plan([10] * 8, 4)[0] == [4] * 8
    rt = Runtime(False, 0, 0, 1, torch.device("cpu"), "cpu")
    sc = StepControl(rt, 100.0)
    assert sc.decide(float("nan"), False)[0] and sc.decide(101.0, False)[0] and not sc.decide(5.0, False)[0]
    assert sc.decide(5.0, True)[1]
    ab = AsyncBoundary("cpu", sync_every=3)
    ab.submit(4, torch.tensor(2.5))
    assert ab.collect() == (4, 2.5) and ab.must_sync(6) and not ab.must_sync(7)


def test_document_selection_rule():
    """Token-id selection rules: length band, typicality band after warm-up, duplicate prefix, start phase."""
    import numpy as np

    from them_bones_b200.data.select import DocRule
    from them_bones_b200.data.synth import PackedRows, SynthLoader, ZipfDocs
    src = ZipfDocs(4096, doc_len=(16, 300), seed=3)
    rule = DocRule.parse("len:32-256,band:0.1-0.9,warm:64,dedup:8,from:0.5", 4096)
    docs = src.docs(200)
    rule.phase = 0.0
    assert all(rule.decide(docs))                                     # before the start phase nothing is dropped
    rule.phase = 0.6
    docs = src.docs(400)
    weird = np.concatenate([[0], 4000 + (np.arange(100) % 90)]).astype(np.int32)   # rare ids only: far from typical
    docs.append(weird)
    keep = rule.decide(docs)
    lens = np.array([len(d) - 1 for d in docs])
    assert not any(k for k, n in zip(keep, lens) if n < 32 or n > 256)
    assert keep[-1] is False
    c = rule.count
    assert c["drop_length"][1] > 0 and c["drop_band"][1] > 0
    assert int(c["docs_read"].sum()) == 601 and "kept" in rule.line()
    dd = DocRule.parse("dedup:8", 4096)
    dd.phase = 1.0
    assert dd.decide([docs[5], docs[6], docs[5].copy()]) == [True, True, False] and dd.count["drop_dup"][1] == 1
    frac = c["docs_kept"][1] / c["docs_read"][1]
    assert 0.4 < frac < 0.9                                           # the band keeps about 80 % of the in-range documents
    # the packer only sees accepted documents and still fills its rows
    ld = SynthLoader(4096, 128, 4, seed=1, doc_len=(16, 300), rule=DocRule.parse("len:64-300", 4096))
    ld.rule.phase = 1.0
    x, y = ld.next_step()
    assert x.shape == (4, 128) and ld.rule.count["drop_length"][1] > 0
    assert isinstance(ld.rows, PackedRows) and ld.rows.rule is ld.rule


def test_native_call_sites_match_the_c_signatures():
    """Every ``call("bones_...", ...)`` in the package and the tests passes as many arguments as the ``extern "C"``
    entry point declares (ctypes does not check, and a short call reads garbage for the missing ones)."""
    import ast
    import glob
    import re
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    sigs = {}
    for f in glob.glob(os.path.join(root, "them_bones_b200", "csrc", "*.cu")):
        src = re.sub(r"//[^\n]*", "", open(f).read())
        for m in re.finditer(r"\bint\s+(bones_\w+)\s*\(([^)]*)\)\s*\{", src):
            args = m.group(2).strip()
            sigs[m.group(1)] = 0 if args in ("", "void") else args.count(",") + 1
    assert len(sigs) > 40
    star = {"aux_ptrs": 5}                                     # helpers that expand to a fixed number of arguments
    seen = 0
    files = glob.glob(os.path.join(root, "them_bones_b200", "**", "*.py"), recursive=True) + \
        glob.glob(os.path.join(root, "tests", "*.py")) + glob.glob(os.path.join(root, "*.py"))
    for f in files:
        for node in ast.walk(ast.parse(open(f).read())):
            if not (isinstance(node, ast.Call) and node.args and isinstance(node.args[0], ast.Constant)
                    and isinstance(node.args[0].value, str) and node.args[0].value.startswith("bones_")):
                continue
            fn = node.func
            if (fn.attr if isinstance(fn, ast.Attribute) else getattr(fn, "id", "")) != "call":
                continue
            n = 0
            for a in node.args[1:]:
                if isinstance(a, ast.Starred):
                    n += star[a.value.func.id]
                else:
                    n += 1
            name = node.args[0].value
            assert name in sigs, f"{f}: {name} is not an entry point of the library"
            assert n == sigs[name], f"{f}:{node.lineno}: {name} takes {sigs[name]} arguments, the call passes {n}"
            seen += 1
    assert seen > 40


def test_micro_batch_follows_the_ranks_share_of_a_fixed_global_batch():
    from them_bones_b200.config import micro_batch_for
    got = [micro_batch_for(524288, w, 64, 2048) for w in (1, 2, 4, 8, 16)]
    assert got == [64, 64, 64, 32, 16]
    assert micro_batch_for(524288, 1, 48, 2048) == 32          # must divide the 256 windows of the step
    assert micro_batch_for(2048, 8, 64, 2048) == 1


def test_mxfp8_linear_statement_trains_like_the_plain_one():
    """The block-scaled projections' PyTorch statement (the CPU path and the GPU kernels' oracle): forward and all three
    gradients stay within quantisation noise of the plain linear."""
    import torch
    from them_bones_b200 import ops
    torch.manual_seed(0)
    x = torch.randn(256, 128, requires_grad=True)
    w = (torch.randn(384, 128) * 0.1).requires_grad_(True)
    g = torch.randn(256, 384)
    ops.linear(x, w, precision="mxfp8").backward(g)
    got = (x.grad.clone(), w.grad.clone())
    x.grad = w.grad = None
    ops.linear(x, w).backward(g)
    rel = lambda a, b: float((a - b).norm() / b.norm())  # noqa: E731
    assert rel(got[0], x.grad) < 0.06 and rel(got[1], w.grad) < 0.06
    q = ops.linear_qkv(x, w[:128], w[128:256], w[256:], precision="mxfp8")
    assert q.shape == (256, 384) and rel(q, x @ w.T) < 0.06


def test_library_ops_have_fake_and_autograd_registrations():
    """The kernels registered with torch.library trace on fake tensors (shapes, dtypes and the autograd graph) without
    running anything: what torch.compile / export need from an op."""
    import torch
    from torch._subclasses.fake_tensor import FakeTensorMode
    from them_bones_b200.ops import registry as R
    assert all(hasattr(torch.ops.bones, n) for n in R.OPS)
    with FakeTensorMode():
        qkv = torch.empty(2, 256, 3 * 2 * 128, dtype=torch.bfloat16, requires_grad=True)
        cos, sin = torch.empty(256, 64), torch.empty(256, 64)
        ds = torch.zeros(2, 256, dtype=torch.int32)
        y = R.attention(qkv, cos, sin, 2, 128, 0.1, ds, 128)
        assert y.shape == (2, 256, 256) and y.dtype == torch.bfloat16 and y.requires_grad
        (g,) = torch.autograd.grad(y.sum(), qkv)
        assert g.shape == qkv.shape
        y2, lse, qk = torch.ops.bones.attention_fwd(qkv, cos, sin, None, 2, 128, 0.1, 0)
        assert lse.shape == (2, 2, 256) and lse.dtype == torch.float32 and not lse.requires_grad and qk.shape == (512, 512)
        x = torch.empty(8, 1280, dtype=torch.bfloat16, requires_grad=True)
        z = R.rms_norm(x)
        assert z.shape == x.shape and torch.autograd.grad(z.sum(), x)[0].shape == x.shape


def test_muon_placement_balances_newton_schulz_work():
    """Every rank's share of the orthogonalisation work with the planned placement against the plain ceil split."""
    from them_bones_b200.optim.lean import plan_muon_counts
    shapes = [(20, 3840, 1280), (20, 1280, 1280), (20, 5120, 1280), (20, 1280, 5120)]
    cost = [max(r, c) * min(r, c) ** 2 for _, r, c in shapes]
    counts = plan_muon_counts(shapes, 8)
    for (n, _, _), c in zip(shapes, counts):
        assert sum(c) == n and max(c) - min(c) <= 1
    load = [sum(counts[g][r] * cost[g] for g in range(4)) for r in range(8)]
    naive = [sum(min(3, max(0, 20 - r * 3)) * cost[g] for g in range(4)) for r in range(8)]
    assert max(load) < 0.87 * max(naive)                 # 10 matrices on the busiest rank instead of 12
    assert max(load) - min(load) <= max(cost)
    assert plan_muon_counts([(4, 64, 64)], 1) == [[4]]
    assert plan_muon_counts([(3, 64, 32)], 4) == [[1, 1, 1, 0]]


def test_local_expert_step_gates_a_non_finite_gradient_per_expert():
    """An expert whose gradient holds a NaN sits the step out (its weights stay finite); the other experts of the same
    stacked parameter step exactly as they would without it; the step is reported as bad without a host read."""
    from them_bones_b200.optim.lean import MuonLocal
    torch.manual_seed(0)
    group = dict(momentum=0.95, beta2=0.95, lr=0.02, weight_decay=0.0, ns_steps=5)
    grads = torch.randn(4, 32, 16)

    def run(poison):
        p = torch.nn.Parameter(torch.randn(4, 32, 16, generator=torch.Generator().manual_seed(1)))
        p.main_grad = grads.clone()
        if poison:
            p.main_grad[2, 3, 5] = float("nan")
        opt = MuonLocal([dict(group, params=[p])], ns_dtype=torch.float32)
        return p, opt.step(1.0)

    clean, bad0 = run(False)
    gated, bad1 = run(True)
    assert not bool(bad0) and bool(bad1)
    assert torch.isfinite(gated).all()
    keep = [0, 1, 3]
    assert torch.allclose(gated[keep], clean[keep], atol=1e-6)
    assert not torch.allclose(gated[2], clean[2], atol=1e-4)      # the poisoned expert did not take the clean step


def _docs(n, lo, hi, seed, vocab=4096):
    from them_bones_b200.data.synth import ZipfDocs
    return ZipfDocs(vocab, doc_len=(lo, hi), seed=seed).docs(n)


def test_pool_mix_reaches_its_share_from_the_decision_on_and_respects_passes():
    """A stored pool mixed into the refills at a token share, from a start fraction on, this rank's documents only, each
    at most ``rep`` times, paid from a token debt (the reference's DSEL lane)."""
    from them_bones_b200.data.streams import PoolMix, doc_hash
    pool = _docs(200, 50, 150, seed=5)
    a = PoolMix(pool, share=0.2, start=0.5, rep=2, rank=0, world=2, seed=3)
    b = PoolMix(pool, share=0.2, start=0.5, rep=2, rank=1, world=2, seed=3)
    assert sorted(a.mine + b.mine) == list(range(200)) and not set(a.mine) & set(b.mine)
    refill = _docs(64, 100, 300, seed=6)
    assert a.mix(refill) == refill                                   # before the decision: untouched
    a.phase = 0.6
    kit = added = 0
    for i in range(6):
        docs = _docs(64, 100, 300, seed=10 + i)
        out = a.mix(docs)
        assert out[:len(docs)] == docs
        kit += sum(len(d) for d in docs)
        added += sum(len(d) for d in out[len(docs):])
        assert all(doc_hash(d, 3) % 2 == 0 for d in out[len(docs):])
    assert abs(added / (kit + added) - 0.2) < 0.02
    many = PoolMix(pool, share=0.9, start=0.0, rep=2, seed=3)
    total = sum(len(many.mix(_docs(64, 100, 300, seed=40 + i))) - 64 for i in range(8))
    assert total == 2 * 200 and many.count["short"] > 0            # every document at most twice, then nothing more


def test_strata_mix_fills_the_stratum_furthest_below_its_first_phase_share():
    from them_bones_b200.data.streams import StrataMix
    pool = _docs(600, 20, 1500, seed=7)
    sm = StrataMix(pool, share=0.3, start=0.5, split=64, seed=1)
    long_docs = _docs(80, 600, 1500, seed=8)
    short_docs = _docs(80, 20, 100, seed=9)
    for _ in range(3):
        assert sm.mix(long_docs + short_docs) == long_docs + short_docs   # phase 1: counted, nothing added
    sm.phase = 0.7
    out = sm.mix(short_docs)                                              # the long strata are now far below their share
    added = out[len(short_docs):]
    assert added and sum(len(d) for d in added) >= 0.3 / 0.7 * sum(len(d) for d in short_docs) - 1500
    assert min(len(d) for d in added) > 512                               # all representatives come from the long buckets
    assert int(sm.rep[0].sum()) == len(added)


def test_masked_blocks_are_never_targets_and_follow_the_late_schedule():
    from them_bones_b200.data.streams import MaskedBlocks, Streams, decode_row
    from them_bones_b200.data.synth import SynthLoader, slice_windows
    import numpy as np
    mb = MaskedBlocks(share=0.1, sep_id=4095, examples=3, context=10, answer=4, late=True, seed=0)
    docs = _docs(64, 100, 300, seed=2)
    early = mb.make(docs)
    mb.phase = 0.9
    late = mb.make(docs)
    assert sum(map(len, late)) > 2 * sum(map(len, early))                 # 0.75 x before 0.8 of the run, 2 x after
    blk = early[0]
    assert blk[0] == 0 and len(blk) == 1 + 3 * (10 + 1 + 4) and int((blk < 0).sum()) == 3 * 11
    ids, train = decode_row(blk)
    assert ids.min() >= 0 and int(train.sum()) == 1 + 3 * 4 and ids[11] == 4095
    row = np.concatenate([blk, docs[0].astype(np.int64), blk])[:129]
    x, y = slice_windows(row, 64, 0)
    assert x.min() >= 0 and x.shape == (2, 64)
    ids, train = decode_row(row)
    flat_y = y.reshape(-1)
    masked_next = ~train[1:129]
    assert (flat_y[masked_next] == -1).all() and (flat_y[~masked_next & (ids[1:129] != 0)] >= 0).all()
    st = Streams.parse("blocks:0.05,edge", vocab=4096, seq_len=128, seed=1)
    ld = SynthLoader(4096, 128, 8, seed=1, doc_len=(16, 300), streams=st)
    for _ in range(6):
        xb, yb = ld.next_step()
        assert int(xb.min()) >= 0 and int(yb.min()) >= -1
    assert st.blocks.count["blocks"] > 0 and st.edge.n["rows"] == 6 and "edge relay" in st.lines()[-1]


def test_edge_relay_keeps_the_tokens_and_moves_the_cuts_to_long_documents():
    """Every window edge cuts some piece; the re-lay keeps every piece whole and chooses long plain documents for the
    cuts: no block and fewer short documents are cut, and the row holds the same pieces."""
    import numpy as np
    from them_bones_b200.data.streams import EdgeRelay, MaskedBlocks
    rng = np.random.default_rng(0)
    er = EdgeRelay(256)
    mb = MaskedBlocks(share=0.5, sep_id=4095, examples=3, context=20, answer=6, seed=1)
    for k in range(12):
        docs = _docs(40, 20, 300, seed=100 + k)
        parts = docs[:14] + mb.make(docs)[:6]
        order = rng.permutation(len(parts))
        row = np.concatenate([np.asarray(parts[i], dtype=np.int64) for i in order])[:8 * 256 + 1]
        out = er.relay(row)
        assert len(out) == len(row)
        pieces = lambda r: sorted(tuple(p) for p in np.split(r, np.flatnonzero(np.where(r < 0, -r - 1, r) == 0)[1:]))  # noqa: E731
        assert pieces(out) == pieces(row)
    b, a = er.split["before"], er.split["after"]
    assert b[2] > 0 and a[2] == 0                                 # blocks were cut before, none after
    assert a[1] < b[1] and er.n["moved"] > 0                      # fewer short documents cut
    assert "edge relay" in er.line()


def test_shared_dedup_drops_across_ranks_with_a_fixed_lag(tmp_path):
    """Two ranks in one process: what rank 1 accepted in batch 0 is dropped on rank 0 from batch 2 on (lag 2), whatever
    the timing; a document repeated on the same rank is dropped at once."""
    from them_bones_b200.data.streams import SharedDedup
    root = str(tmp_path / "dd")
    r0 = SharedDedup(root, 0, 2, bits=16, wait_s=5.0)
    r1 = SharedDedup(root, 1, 2, bits=16, wait_s=5.0)
    docs = _docs(12, 30, 60, seed=11)
    for b in range(4):
        for r in (r0, r1):                                             # rank 0 first: it only needs slots of batch b - 2
            if r is r1 and b >= 2:
                continue
            r.begin_batch(b)
        if b == 0:
            assert r0.decide(docs[:4] + docs[:1]) == [True] * 4 + [False]
            assert r1.decide(docs[4:8]) == [True] * 4
        elif b == 1:
            assert r0.decide(docs[4:6]) == [True, True]               # rank 1's batch 0 is not merged yet
            assert r1.decide(docs[8:10]) == [True, True]
        elif b == 2:
            assert r0.decide(docs[6:8]) == [False, False]             # merged now
            r1.begin_batch(b)
            assert r1.decide(docs[0:2]) == [False, False]
        else:
            r1.begin_batch(b)
            assert r0.decide(docs[8:10]) == [False, False] and r1.decide(docs[10:12]) == [True, True]
        r0.end_batch()
        r1.end_batch()
    assert r0.n["merged_hashes"] == 4 + 4 + 2 + 2


def test_local_expert_stacks_alias_parameters_and_restore_state():
    """The stacked expert optimizer keeps every parameter, its gradient and its optimizer state as views of one stack per
    shape; restoring a checkpointed state writes through those views (the stack stays the single copy)."""
    from them_bones_b200.optim.lean import MuonLocal
    torch.manual_seed(0)
    group = dict(momentum=0.95, beta2=0.95, lr=0.02, weight_decay=0.0, ns_steps=5)
    ps = [torch.nn.Parameter(torch.randn(4, 64, 32).bfloat16()), torch.nn.Parameter(torch.randn(4, 32, 64).bfloat16()),
          torch.nn.Parameter(torch.randn(2, 64, 32).bfloat16())]
    before = [p.detach().clone() for p in ps]
    opt = MuonLocal([dict(group, params=ps)], native=True)
    assert len(opt.stacks) == 2 and sorted(st.n for st in opt.stacks) == [4, 6]
    for p, b in zip(ps, before):
        assert torch.equal(p.detach(), b) and p.main_grad.shape == p.shape and p.main_grad.dtype == torch.float32
    st = next(s for s in opt.stacks if s.n == 6)
    assert ps[0].data_ptr() == st.W.data_ptr() and ps[2].data_ptr() == st.W[4:].data_ptr()
    ps[2].main_grad.fill_(3.0)
    assert float(st.G[4:].min()) == 3.0 and float(st.G[:4].abs().max()) == 0.0
    opt.zero_grad()
    assert float(st.G.abs().max()) == 0.0
    saved = {k: torch.full_like(v, 0.5) for k, v in opt.state[ps[2]].items()}
    opt.load_state(ps[2], saved)
    assert float(st.master[4:].min()) == 0.5 and float(st.momentum[4:].max()) == 0.5 and float(ps[2].detach().float().min()) == 0.5
    assert torch.equal(st.master[:4], before[0].float())              # the other parameter of the stack is untouched
