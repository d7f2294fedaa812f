"""MoE blocks and hashed tables on the GPU: native kernels against the plain-PyTorch path on the same weights."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _rel(a, b):
    return float((a.float() - b.float()).norm() / b.float().norm().clamp_min(1e-12))


def test_moe_block_native_matches_reference_path():
    from them_bones_b200 import ops
    from them_bones_b200.config import GPTConfig
    from them_bones_b200.models.gpt import GPT
    from them_bones_b200.ops import _lib as L
    cfg = GPTConfig(sequence_len=256, vocab_size=2048, n_layer=2, n_head=2, n_embd=256, head_dim=128, doc_mask=True,
                    moe_layers=(1,), moe_experts=4, moe_topk=2, moe_capacity=160, moe_hidden=256, moe_shared=256)
    torch.manual_seed(0)
    model = GPT(cfg)
    model.init_weights()
    with torch.no_grad():
        for blk in model.transformer.h:
            blk.attn.c_proj.weight.normal_(0, 0.02)
        model.transformer.h[0].mlp.c_proj.weight.normal_(0, 0.02)
        moe = model.transformer.h[1].mlp
        moe.w_proj.normal_(0, 0.02)
        moe.shared.c_proj.weight.normal_(0, 0.02)
        model.lm_head.weight.normal_(0, 0.05)
    model = model.cuda().cast_compute(torch.bfloat16)
    x = torch.randint(1, cfg.vocab_size, (2, 256), device="cuda")
    x[:, 0] = 0
    y = torch.roll(x, -1, 1)
    outs = {}
    for name, ref in (("ref", True), ("native", False)):
        ops.set_reference_path(ref)
        for p in model.parameters():
            p.grad = None
        loss, stats = model(x, y)
        loss.backward()
        outs[name] = (float(loss), {n: p.grad.float().clone() for n, p in model.named_parameters() if p.grad is not None}, stats)
    ops.set_reference_path(False)
    torch.cuda.synchronize()
    L.check_error_word()
    assert abs(outs["ref"][0] - outs["native"][0]) < 2e-2 * abs(outs["ref"][0])
    assert ops.COUNTS["moe_experts"] > 0 and ops.COUNTS["moe_dispatch"] > 0 and ops.COUNTS["moe_combine"] > 0
    for n in ("transformer.h.1.mlp.w_fc", "transformer.h.1.mlp.w_proj", "transformer.h.1.mlp.router",
              "transformer.h.1.mlp.shared.c_fc.weight", "transformer.h.0.attn.c_q.weight"):
        assert _rel(outs["native"][1][n], outs["ref"][1][n]) < 8e-2, (n, _rel(outs["native"][1][n], outs["ref"][1][n]))


def test_trainer_with_moe_and_tables_steps_on_gpu():
    from them_bones_b200 import ops
    from them_bones_b200.config import GPTConfig, Hyper
    from them_bones_b200.data.synth import SynthLoader
    from them_bones_b200.ops import _lib as L
    from them_bones_b200.runtime import Runtime
    from them_bones_b200.trainer import Trainer
    rt = Runtime(False, 0, 0, 1, torch.device("cuda", 0), "cuda")
    cfg = GPTConfig(sequence_len=256, vocab_size=2048, n_layer=2, n_head=2, n_embd=256, head_dim=128, doc_mask=True,
                    moe_layers=(1,), moe_experts=4, moe_topk=2, moe_capacity=160, moe_hidden=256,
                    table_orders=(2, 3), table_rows=1 << 14)
    hy = Hyper()
    hy.total_batch, hy.device_batch = 4 * 256, 4
    tr = Trainer(cfg, hy, rt, horizon_steps=10)
    ld = SynthLoader(cfg.vocab_size, 256, tr.local_windows, seed=0, doc_len=(32, 256), pin=True)
    losses = []
    for _ in range(6):
        x, y = ld.next_step()
        losses.append(float(tr.train_step(x, y)))
    torch.cuda.synchronize()
    L.check_error_word()
    assert all(l == l for l in losses) and losses[-1] < losses[0]
    st = tr.tables.exchange.read_stats()                     # the peer-memory table path, here on a one-entry peer list
    assert st["touched"] > 0 and st["skipped"] == 0 and st["overflow"] == 0
    assert float(tr.tables.shards[0].float().abs().sum()) > 0


@pytest.mark.parametrize("opt", ["rowrms", "adam"])
def test_native_table_push_and_update_match_the_statement(opt):
    """Gradient rows pushed into the owner's staging buffer, duplicates summed in sorted order, the table updated in
    place: against the PyTorch statement of the same step (bf16 rows are rounded stochastically, so one bf16 step of
    slack per element)."""
    from them_bones_b200.models.tables import HashedTables
    from them_bones_b200.ops import _lib as L
    from them_bones_b200.parallel.symm import SoloComm
    from them_bones_b200.ref import functional as RF
    from them_bones_b200.runtime import Runtime
    rt = Runtime(False, 0, 0, 1, torch.device("cuda", 0), "cuda")
    torch.manual_seed(0)
    rows, dim, n = 4096, 256, 3000
    tab = HashedTables((2,), rows, dim, device="cuda", dtype=torch.bfloat16, opt=opt, decay=1e-3)
    tab.exchange = SoloComm(rt).table_exchange(tab, entries_per_step=n)
    assert tab.exchange.native
    tab.shards[0].copy_(torch.randn(rows, dim, device="cuda") * 0.1)
    before = tab.shards[0].float().clone()
    ids = torch.randint(0, 200, (n,), device="cuda")          # many duplicates per row
    ids[:50] = torch.arange(3000, 3050, device="cuda")        # and some rows touched once
    g = (torch.randn(n, dim, device="cuda") * 0.01).bfloat16()
    tab.record_grad(0, ids[:1000], g[:1000])                  # pushed in several pieces, as the micro-steps do
    tab.record_grad(0, ids[1000:], g[1000:])
    tab.step(0.02)
    torch.cuda.synchronize()
    L.check_error_word()
    st = tab.exchange.read_stats()
    uniq, inv = torch.unique(ids, return_inverse=True)
    assert st["touched"] == len(uniq) and st["skipped"] == 0 and st["overflow"] == 0
    acc = torch.zeros(len(uniq), dim, device="cuda").index_add_(0, inv, g.float())
    want = before.clone()
    if opt == "rowrms":
        sq = torch.zeros(rows, device="cuda")
        RF.table_rowrms_update(want, uniq, acc, sq, lr=0.02, beta=0.99, eps=1e-8, decay=1e-3)
        assert torch.allclose(tab.row_sq[0], sq, rtol=1e-4, atol=1e-12)
    else:
        m, v = torch.zeros(len(uniq), dim, device="cuda"), torch.zeros(len(uniq), dim, device="cuda")
        w = want.index_select(0, uniq)
        m.lerp_(acc, 0.1); v.lerp_(acc.square(), 0.01)
        w = w * (1 - 0.02 * 1e-3) - 0.02 * (m / 0.1) / ((v / 0.01).sqrt() + 1e-8)
        want.index_copy_(0, uniq, w)
    got = tab.shards[0].float()
    untouched = torch.ones(rows, dtype=torch.bool, device="cuda")
    untouched[uniq] = False
    assert torch.equal(got[untouched], before[untouched])
    ulp = want.abs().clamp_min(1e-6) * 2.0 ** -7
    assert bool(((got - want).abs() <= ulp).all()), float(((got - want).abs() / ulp).max())
    # a second step meets a clean staging buffer
    tab.record_grad(0, ids[:10], g[:10])
    tab.step(0.02)
    assert tab.exchange.read_stats()["touched"] == len(uniq) + len(torch.unique(ids[:10]))


def test_native_newton_schulz_matches_reference():
    from them_bones_b200.ops import _lib as L
    from them_bones_b200.ops import muon_native as MN
    from them_bones_b200.ref import functional as RF
    torch.manual_seed(0)
    for shape in ((3, 512, 256), (2, 256, 512), (2, 256, 256)):
        x = torch.randn(*shape, device="cuda")
        x = (x / (x.norm(dim=(-2, -1), keepdim=True) * 1.01 + 1e-6)).bfloat16().contiguous()
        got = MN.newton_schulz(x, 5)
        ref = RF.newton_schulz(x.float(), 5)
        torch.cuda.synchronize()
        L.check_error_word()
        assert _rel(got, ref) < 5e-2, (shape, _rel(got, ref))


def test_native_slotting_matches_reference():
    from them_bones_b200.ops import cuda as C
    from them_bones_b200.ref import functional as RF
    torch.manual_seed(3)
    for (b, t, e, k, cap) in ((3, 512, 16, 2, 40), (2, 2048, 16, 2, 320), (4, 300, 8, 1, 20)):
        logits = torch.randn(b * t, e, device="cuda")
        _, idx, _ = RF.moe_route(logits, k)
        slot_r, tok_r = RF.moe_slots(idx, b, t, e, cap)
        slot_n, tok_n = C.moe_slots(idx, b, t, e, cap)
        torch.cuda.synchronize()
        assert torch.equal(slot_n, slot_r) and torch.equal(tok_n, tok_r), (b, t, e, k, cap)
        if cap <= 40:
            assert (slot_r == e * b * cap).any()                # some assignments were dropped: the cap was exercised


def test_native_decode_with_moe_blocks_and_tables_matches_the_cached_route():
    """The CUDA-graph decode step on a model with routed experts and hashed input tables: logits of every step against
    the PyTorch KV-cache route fed the same tokens, then a whole greedy decode (graph replays) against eager stepping of
    the same kernels."""
    from them_bones_b200.config import GPTConfig
    from them_bones_b200.models.gpt import GPT
    from them_bones_b200.models.tables import HashedTables
    from them_bones_b200.ops import _lib as L
    from them_bones_b200.utils import decode as D
    cfg = GPTConfig(sequence_len=512, vocab_size=4096, n_layer=3, n_head=2, n_embd=256, head_dim=128, doc_mask=True,
                    moe_layers=(1, 2), moe_experts=4, moe_topk=2, moe_capacity=160, moe_hidden=256,
                    table_orders=(2, 3), table_rows=1 << 12)
    torch.manual_seed(0)
    model = GPT(cfg)
    model.init_weights()
    with torch.no_grad():
        for blk in model.transformer.h:
            blk.attn.c_proj.weight.normal_(0, 0.02)
        model.transformer.h[0].mlp.c_proj.weight.normal_(0, 0.02)
        for i in (1, 2):
            model.transformer.h[i].mlp.w_proj.normal_(0, 0.02)
        model.lm_head.weight.normal_(0, 0.05)
    model = model.cuda().cast_compute(torch.bfloat16).eval()
    tables = HashedTables(cfg.table_orders, cfg.table_rows, cfg.n_embd, seed=cfg.table_seed, device="cuda", dtype=torch.bfloat16)
    for sh in tables.shards:
        sh.copy_(torch.randn_like(sh) * 0.3)
    model.attach_tables(tables)
    assert D.NativeDecoder.eligible(model)
    torch.manual_seed(5)
    b, p, n_new = 4, 40, 12
    prompts = torch.randint(1, cfg.vocab_size, (b, p), device="cuda")
    prompts[:, 0] = 0
    prompts[1, 33] = 0
    with torch.no_grad():
        ca, cb = D.KVCache(model, b, p + n_new), D.KVCache(model, b, p + n_new)
        la = D._forward_cached(model, prompts, ca)
        D._forward_cached(model, prompts, cb)
        tok = la.argmax(-1)
        out = torch.zeros(b, p + n_new, dtype=torch.int64, device="cuda")
        out[:, :p] = prompts
        dec = D.NativeDecoder(model, cb, tok, out)
        for s in range(5):
            out[:, p + s] = tok                           # the history the table hashes read
            ref = D._forward_cached(model, tok[:, None], ca)
            dec.tok.copy_(tok)
            dec._step()
            got = dec.last_logits[:, :cfg.vocab_size].float()
            assert _rel(got, ref) < 4e-2, (s, _rel(got, ref))
            tok = ref.argmax(-1)
        torch.cuda.synchronize()
        L.check_error_word()
        full = D.greedy_decode(model, prompts, n_new)
        cc = D.KVCache(model, b, p + n_new)
        out2 = torch.zeros_like(full)
        out2[:, :p] = prompts
        dec2 = D.NativeDecoder(model, cc, prompts[:, 0], out2, prompt_len=p)
        for _ in range(p + n_new - 1):
            dec2._step()
        torch.cuda.synchronize()
    assert torch.equal(full, out2) and torch.equal(full[:, :p], prompts)


def test_local_expert_stack_matches_per_parameter_update():
    """The stacked expert optimizer (fused prologue, one batched tcgen05 Newton-Schulz per shape, native update) against
    the per-parameter PyTorch statement of the same Muon step on the same gradients; then a non-finite gradient entry is
    dropped, the step is reported, and the weights stay finite."""
    from them_bones_b200.optim.lean import MuonLocal
    group = dict(momentum=0.95, beta2=0.95, lr=0.02, weight_decay=0.01, ns_steps=5)

    def make():
        g = torch.Generator(device="cuda").manual_seed(1)
        shapes = [(4, 256, 128), (4, 256, 128), (4, 128, 256)]
        return [torch.nn.Parameter((torch.randn(*s, device="cuda", generator=g) * 0.05).bfloat16()) for s in shapes]

    a, b = make(), make()
    start = [p.detach().float().clone() for p in a]
    oa = MuonLocal([dict(group, params=a)], native=True)
    ob = MuonLocal([dict(group, params=b)], native=False)
    assert len(oa.stacks) == 2 and not ob.stacks
    for p in b:
        p.main_grad = torch.zeros_like(p, dtype=torch.float32)
    gen = torch.Generator(device="cuda").manual_seed(2)
    for _ in range(3):
        for pa, pb in zip(a, b):
            g = torch.randn(pa.shape, device="cuda", generator=gen)
            pa.main_grad.copy_(g)
            pb.main_grad.copy_(g)
        bad_a, bad_b = oa.step(0.5), ob.step(0.5)
        assert not bool(bad_a) and not bool(bad_b)
    for pa, pb, p0 in zip(a, b, start):
        da, db = pa.detach().float() - p0, pb.detach().float() - p0
        rel = float((da - db).norm() / db.norm())
        assert rel < 5e-2, rel
        ma, mb = oa.state[pa]["master"], ob.state[pb]["master"]
        assert float((ma - mb).norm() / (mb - p0).norm()) < 5e-2
    a[0].main_grad[1, 3, 5] = float("nan")
    assert bool(oa.step(0.5))
    assert all(torch.isfinite(p).all() for p in a)
