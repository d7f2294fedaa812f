"""The output-side table's native kernels and loss head against the plain-PyTorch fp32 statement of the same ops."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _rel(a, b):
    return float((a.float() - b.float()).norm() / b.float().norm().clamp_min(1e-12))


def test_signs_gate_and_row_step_kernels_match_reference():
    from them_bones_b200 import ops
    from them_bones_b200.ops import _lib as L
    from them_bones_b200.ref import functional as RF
    torch.manual_seed(0)
    n, dim, v = 1000, 128, 4096
    hs = torch.randint(-(1 << 62), 1 << 62, (n,), device="cuda", dtype=torch.int64)
    rows = torch.randn(n, dim, device="cuda", dtype=torch.bfloat16)
    want = RF.os1_signs(hs, dim) * rows.float()
    assert torch.equal(ops.os1_apply_signs(rows, hs).float(), want)
    g32 = torch.randn(n, dim, device="cuda")
    assert torch.equal(ops.os1_apply_signs(g32, hs), RF.os1_signs(hs, dim) * g32)
    # gate
    b, t = 4, 250
    code = RF.os1_codebook(v, dim, 5).cuda().bfloat16()
    u = (torch.randn(b * t, dim, device="cuda") * 0.3).bfloat16()
    idx = torch.randint(0, v, (b, t), device="cuda")
    got = ops.os1_gate(u, code, idx, 1.0, 32, 0.3, 30.0)
    ref = RF.os1_gate(u, code, idx, 1.0, 32, 0.3, 30.0)
    assert got.shape == (b, t) and float((got - ref).abs().max()) < 2e-3
    # row step, both table dtypes, duplicate-free row list, one zero gradient
    for dt, tol in ((torch.float32, 1e-5), (torch.bfloat16, 5e-3)):
        table = (torch.randn(512, dim, device="cuda") * 0.4).to(dt)
        pick = torch.randperm(512, device="cuda")[:200]
        g = torch.randn(200, dim, device="cuda") * 1e-5
        g[7] = 0
        want = RF.os1_row_step(table[pick], g, 0.125, 1e-12, 4.0)
        keep = table.clone()
        capped = ops.os1_row_step(table, pick, g, lr=0.125, eps=1e-12, cap=4.0)
        assert _rel(table[pick], want) < tol
        mask = torch.ones(512, dtype=torch.bool, device="cuda")
        mask[pick] = False
        assert torch.equal(table[mask], keep[mask])
        stepped = keep[pick].float() - g * (0.125 / (g.square().mean(1, keepdim=True).sqrt() + 1e-12))
        assert abs(int(capped) - int((stepped.square().mean(1).sqrt() > 0.5).sum())) <= 2
    L.check_error_word()


@pytest.mark.parametrize("vocab,vp,m", [(4096, 4096, 600), (50304, 50432, 4500)])
def test_os1_loss_head_matches_reference(vocab, vp, m):
    from them_bones_b200 import ops
    from them_bones_b200.ops import _lib as L
    from them_bones_b200.ref import functional as RF
    torch.manual_seed(1)
    d, dim = 256, 128
    kw = dict(a0=1.0, glin=0.01, beta=3.0, thr=0.7)
    x = torch.randn(m, d, device="cuda", dtype=torch.bfloat16)
    w = (torch.randn(vp, d, device="cuda") * 0.05).bfloat16()
    code = RF.os1_codebook(vp, dim, 3).cuda().bfloat16()
    u = (torch.randn(m, dim, device="cuda") * 0.35).bfloat16()
    gate = torch.rand(m, device="cuda")
    tg = torch.randint(0, vocab, (m,), device="cuda")
    tg[::17] = -1
    xn, wn, un = x.clone().requires_grad_(), w.clone().requires_grad_(), u.clone().requires_grad_()
    loss = ops.lmhead_loss_os1(xn, wn, tg, vocab, 15.0, un, code, gate, loss_div=2.0, **kw)
    loss.backward()
    xr, wr, ur = x.float().requires_grad_(), w.float().requires_grad_(), u.float().requires_grad_()
    ref = RF.softcap_cross_entropy_os1(xr, wr, tg, vocab, 15.0, ur, code.float(), gate, **kw) / 2.0
    ref.backward()
    L.check_error_word()
    assert abs(float(loss) - float(ref)) < 3e-3 * abs(float(ref))
    assert _rel(xn.grad, xr.grad) < 3e-2 and _rel(wn.grad, wr.grad) < 3e-2 and _rel(un.grad, ur.grad) < 3e-2
    # the thresholded term is live in this test: it moves the loss
    plain = RF.softcap_cross_entropy(x.float(), w.float(), tg, vocab, 15.0) / 2.0
    assert abs(float(plain) - float(ref)) > 1e-3
    # evaluation forms
    with torch.no_grad():
        nll = ops.lmhead_loss_os1(x, w, tg, vocab, 15.0, u, code, gate, reduction="none", **kw)
        nll_r = RF.softcap_cross_entropy_os1(x.float(), w.float(), tg, vocab, 15.0, u.float(), code.float(), gate,
                                             reduction="none", **kw)
        assert _rel(nll, nll_r) < 5e-3
        lg = ops.lmhead_logits_os1(x[:300], w, vocab, 15.0, u[:300], code, gate[:300], **kw)
        ops.set_reference_path(True)
        try:
            lg_r = ops.lmhead_logits_os1(x[:300].float(), w.float(), vocab, 15.0, u[:300].float(), code.float(), gate[:300], **kw)
        finally:
            ops.set_reference_path(False)
        assert lg.shape == (300, vocab) and _rel(lg, lg_r) < 1e-2


def test_model_with_output_table_trains_like_the_reference_path():
    from them_bones_b200 import ops
    from them_bones_b200.config import GPTConfig, Hyper
    from them_bones_b200.data.synth import SynthLoader
    from them_bones_b200.ops import _lib as L
    from them_bones_b200.runtime import Runtime
    from them_bones_b200.trainer import Trainer
    cfg = GPTConfig(sequence_len=256, vocab_size=8192, n_layer=2, n_head=2, n_embd=256, head_dim=128, doc_mask=True,
                    os1_rows=1 << 14, os1_order=2)
    rt = Runtime(False, 0, 0, 1, torch.device("cuda", 0), "cuda")

    def run(ref):
        ops.set_reference_path(ref)
        try:
            h = Hyper()
            h.total_batch, h.device_batch = 8 * 256, 4
            tr = Trainer(cfg, h, rt, optimizer_kind="lean", horizon_steps=8)
            ld = SynthLoader(cfg.vocab_size, 256, tr.local_windows, seed=0, doc_len=(64, 256))
            x, y = ld.next_step()
            out = [float(tr.train_step(x.long(), y)) for _ in range(8)]       # the same windows: the table's rows recur
            return out, tr.os1.stats, tr.os1.shard.float().square().mean(1).sqrt().max()
        finally:
            ops.set_reference_path(False)

    native, st, rmax = run(False)
    L.check_error_word()
    refp, st_r, _ = run(True)
    assert st["updates"] == 8 and st["touched"] == st_r["touched"] > 0
    assert float(rmax) <= cfg.os1_lr * 4.0 * 1.01
    assert native[-1] < native[0] - 1.0
    for a, b in zip(native, refp):
        assert abs(a - b) < 0.03 * abs(b), (native, refp)


def test_packed_views_and_stochastic_rounding_on_device():
    from them_bones_b200.ref import functional as RF
    torch.manual_seed(0)
    m = (torch.randn(64, 128) * 0.3).bfloat16()
    m[3] = 0
    for bits in (1, 4):
        md = m.cuda()
        dev = RF.table_view(md, bits)
        assert dev.dtype == torch.bfloat16 and float(dev[3].abs().sum()) == 0
        # reductions run in another order on the device: the scale may differ from the CPU's by one bf16 step
        assert torch.allclose(dev.cpu().float(), RF.table_view(m, bits).float(), rtol=1e-2, atol=1e-3)
        pk, sc = RF.table_pack_view(md, bits)
        assert pk.dtype == torch.uint8 and pk.shape == (64, 128 * bits // 8)
        assert torch.allclose(RF.table_unpack_view(pk, sc, bits), dev.float(), rtol=4e-3, atol=1e-6)   # packed = the view
        if bits == 1:
            assert torch.equal(pk.cpu(), RF.table_pack_view(m, bits)[0])
    x = torch.full((1 << 20,), 1.0 + 2.0 ** -10, device="cuda")
    y = RF.stochastic_round_bf16(x).float()
    assert set(y.unique().tolist()) == {1.0, 1.0 + 2.0 ** -7} and abs(float(y.mean()) - float(x[0])) < 5e-5
