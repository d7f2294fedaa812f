"""CPU tests of the model family: tiny dense decoder training (benchmark configuration 1), optimizer-class parity,
causality, checkpoint round trip, cached decoding, MoE routing semantics and hashed tables."""
import os

import pytest
import torch

from them_bones_b200.config import GPTConfig, Hyper, model_config_dict
from them_bones_b200.data.synth import SynthLoader
from them_bones_b200.models.gpt import GPT
from them_bones_b200.ref import functional as RF
from them_bones_b200.runtime import Runtime
from them_bones_b200.trainer import Trainer

RT = Runtime(False, 0, 0, 1, torch.device("cpu"), "cpu")


def tiny_cfg(**kw):
    base = dict(sequence_len=256, vocab_size=8192, n_layer=4, n_head=4, n_embd=256, rope_base=10000.0, doc_mask=True)
    base.update(kw)
    return GPTConfig(**base)


def run_steps(cfg, kind, steps=20, seq=256, batch=8, seed=0):
    h = Hyper()
    h.total_batch, h.device_batch = batch * seq, batch
    tr = Trainer(cfg, h, RT, optimizer_kind=kind, horizon_steps=steps)
    ld = SynthLoader(cfg.vocab_size, seq, tr.local_windows, seed=seed, doc_len=(64, 256))
    losses = []
    for _ in range(steps):
        x, y = ld.next_step()
        losses.append(float(tr.train_step(x.long(), y)))
    return tr, losses


def test_config1_tiny_dense_trains_and_optimizers_agree():
    """4 layers x 256, 4 heads x 64, vocab 8192, seq 256, batch 8, Zipf(1.1) tokens, Muon + AdamW, 20 steps."""
    cfg = tiny_cfg()
    _, single = run_steps(cfg, "single")
    _, lean = run_steps(cfg, "lean")
    assert single[0] == pytest.approx(9.01, abs=0.05)             # ln(8192) at init
    assert single[-1] < single[0] - 2.0
    assert all(abs(a - b) < 1e-4 for a, b in zip(single, lean))


def test_causality_and_doc_mask():
    from them_bones_b200.utils.evalbpb import causality_check
    torch.manual_seed(0)
    model = GPT(tiny_cfg(n_layer=2))
    model.init_weights()
    with torch.no_grad():
        for blk in model.transformer.h:
            blk.attn.c_proj.weight.normal_(0, 0.05)
            blk.mlp.c_proj.weight.normal_(0, 0.05)
        model.lm_head.weight.normal_(0, 0.05)
    out = causality_check(model, 8192, 2, 64, "cpu")
    assert out["passed"], out
    # a document does not see the previous one: changing tokens before a BOS leaves later logits unchanged
    x = torch.randint(1, 8192, (1, 64))
    x[0, 0] = 0
    x[0, 32] = 0
    x2 = x.clone()
    x2[0, 1:32] = torch.randint(1, 8192, (31,))
    with torch.no_grad():
        a, b = model(x), model(x2)
    assert float((a[:, 32:] - b[:, 32:]).abs().max()) < 1e-5
    assert float((a[:, 1:32] - b[:, 1:32]).abs().max()) > 1e-4


def test_extras_unet_value_embeds_window_run_and_train():
    cfg = tiny_cfg(n_layer=4, unet=True, value_embeds=2, attn_window=128, attn_long=(3,))
    tr, losses = run_steps(cfg, "lean", steps=6)
    assert losses[-1] < losses[0]
    names = dict(tr.model.named_parameters())
    assert "skip_lambda" in names and "value_embeds.3.weight" in names and "transformer.h.1.ve_lambda" in names


def test_checkpoint_roundtrip_and_inference_wrapper(tmp_path):
    import inference
    from them_bones_b200.utils import ckpt as CK
    cfg = tiny_cfg(n_layer=2)
    tr, _ = run_steps(cfg, "lean", steps=2)
    path = str(tmp_path / "final.pt")
    CK.save_checkpoint(path, tr.model, dict(steps=2), optimizer=tr.optimizer)
    raw = torch.load(path, weights_only=True)
    assert set(raw) == {"model_state", "model_config", "meta"}
    assert raw["model_config"] == model_config_dict(cfg)
    assert "transformer.h.0.attn.c_q.weight" in raw["model_state"] and "lm_head.weight" in raw["model_state"]
    w = inference.load_for_eval(path, "cpu")
    x = torch.randint(1, 8192, (2, 48))
    with torch.no_grad():
        assert torch.allclose(w(x), tr.model(x), atol=1e-5)
    assert w.get_eval_worker() == (int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1)))
    ctx, tot = torch.tensor([10, 20]), torch.tensor([30, 48])
    sc = w.score(x, ctx, tot)
    assert sc.shape == (2,) and (sc < 0).all()


def test_cached_greedy_decode_matches_full_recompute():
    from them_bones_b200.utils.decode import greedy_decode, greedy_decode_full
    torch.manual_seed(1)
    model = GPT(tiny_cfg(n_layer=2, attn_window=128, attn_long=(1,)))
    model.init_weights()
    with torch.no_grad():
        for blk in model.transformer.h:
            blk.attn.c_proj.weight.normal_(0, 0.05)
            blk.mlp.c_proj.weight.normal_(0, 0.05)
        model.lm_head.weight.normal_(0, 0.3)
    model.eval()
    prompts = torch.randint(1, 8192, (3, 20))
    prompts[:, 0] = 0
    prompts[1, 10] = 0
    a = greedy_decode(model, prompts, 12)
    b = greedy_decode_full(model, prompts, 12)
    assert a.shape == (3, 32) and (a == b).all()


def test_bpb_eval_runs():
    from them_bones_b200.utils.evalbpb import evaluate_bpb
    model = GPT(tiny_cfg(n_layer=1))
    model.init_weights()
    out = evaluate_bpb(model, 8192, 2, 128, torch.device("cpu"), max_tokens=512)
    assert out["num_tokens"] >= 256 and 2.0 < out["val_bpb"] < 12.0


# -- MoE -------------------------------------------------------------------------------------------------------------
def test_moe_routing_semantics():
    torch.manual_seed(0)
    logits = torch.randn(12, 4)
    logits[3] = torch.tensor([1.0, 1.0, 0.0, 0.0])             # tie -> lower index first
    p, idx, gates = RF.moe_route(logits, 2)
    assert idx[3].tolist() == [0, 1]
    assert torch.allclose(gates.sum(1), torch.ones(12))
    _, idx1, g1 = RF.moe_route(logits, 1)
    assert torch.allclose(g1[:, 0], p.max(1).values)
    # capacity is counted left to right inside each sequence
    idx = torch.tensor([[0], [0], [0], [1], [0], [0]])          # b=2, t=3
    slot, tok = RF.moe_slots(idx, 2, 3, 2, 2)
    total = 2 * 2 * 2
    assert slot.view(-1).tolist() == [0, 1, total, 6, 2, 3]      # third token of row 0 is dropped
    assert tok.tolist() == [0, 1, 4, 5, 6, 6, 3, 6]


def test_moe_layer_matches_dense_loop_and_trains():
    cfg = tiny_cfg(n_layer=2, n_embd=64, n_head=2, vocab_size=512, sequence_len=64, moe_layers=(1,), moe_experts=4,
                   moe_topk=2, moe_capacity=64, moe_hidden=32, moe_shared=32)
    torch.manual_seed(0)
    model = GPT(cfg)
    model.init_weights()
    moe = model.transformer.h[1].mlp
    with torch.no_grad():
        moe.w_proj.normal_(0, 0.1)
        moe.shared.c_proj.weight.normal_(0, 0.1)
    x = torch.randn(2, 64, 64)
    out = moe(x)
    # capacity 64 never drops: compare with a per-token loop over its two experts
    h = x.reshape(-1, 64)
    p, idx, gates = RF.moe_route(torch.nn.functional.linear(h, moe.router), 2)
    ref = torch.zeros_like(h)
    for n in range(h.shape[0]):
        for k in range(2):
            e = int(idx[n, k])
            ref[n] += gates[n, k] * RF.mlp(h[n:n + 1], moe.w_fc[e], moe.w_proj[e])[0]
    ref = ref + RF.mlp(h, moe.shared.c_fc.weight, moe.shared.c_proj.weight)
    assert torch.allclose(out.reshape(-1, 64), ref, atol=1e-5)
    hy = Hyper()
    hy.total_batch, hy.device_batch = 4 * 64, 4
    tr = Trainer(cfg, hy, RT, optimizer_kind="lean", horizon_steps=8)
    ld = SynthLoader(512, 64, tr.local_windows, seed=0, doc_len=(16, 64))
    losses = []
    for _ in range(8):
        xb, yb = ld.next_step()
        losses.append(float(tr.train_step(xb.long(), yb)))
    assert losses[-1] < losses[0] and tr.last_moe_stats is not None and tr.last_moe_stats.shape == (1, 3 + 4)


def test_moe_capacity_is_causal():
    cfg = tiny_cfg(n_layer=1, n_embd=64, n_head=2, vocab_size=512, sequence_len=64, moe_layers=(0,), moe_experts=4,
                   moe_topk=1, moe_capacity=4, moe_hidden=32, doc_mask=False)
    torch.manual_seed(0)
    model = GPT(cfg)
    model.init_weights()
    with torch.no_grad():
        model.transformer.h[0].attn.c_proj.weight.normal_(0, 0.05)
        model.transformer.h[0].mlp.w_proj.normal_(0, 0.2)
        model.lm_head.weight.normal_(0, 0.1)
    from them_bones_b200.utils.evalbpb import causality_check
    assert causality_check(model, 512, 2, 64, "cpu")["passed"]


# -- tables ----------------------------------------------------------------------------------------------------------
def test_ngram_hash_is_causal_and_deterministic():
    idx = torch.randint(1, 1000, (2, 32))
    a = RF.ngram_rows(idx, 3, 1 << 16, seed=5)
    b = RF.ngram_rows(idx, 3, 1 << 16, seed=5)
    assert (a == b).all() and a.min() >= 0 and a.max() < (1 << 16)
    idx2 = idx.clone()
    idx2[:, 20:] = 7
    assert (RF.ngram_rows(idx2, 3, 1 << 16, seed=5)[:, :20] == a[:, :20]).all()
    assert len(torch.unique(a)) > 50
    assert (RF.ngram_rows(idx, 2, 1 << 16, seed=5) != a).any()


def test_tables_zero_init_is_identity_then_learns():
    cfg0 = tiny_cfg(n_layer=1, n_embd=64, n_head=2, vocab_size=512, sequence_len=64)
    cfg1 = tiny_cfg(n_layer=1, n_embd=64, n_head=2, vocab_size=512, sequence_len=64, table_orders=(2, 3), table_rows=1 << 12)
    hy = Hyper()
    hy.total_batch, hy.device_batch = 4 * 64, 4
    tr0 = Trainer(cfg0, hy, RT, optimizer_kind="lean", horizon_steps=10)
    tr1 = Trainer(cfg1, hy, RT, optimizer_kind="lean", horizon_steps=10)
    ld0 = SynthLoader(512, 64, 4, seed=0, doc_len=(16, 64))
    ld1 = SynthLoader(512, 64, 4, seed=0, doc_len=(16, 64))
    x0, y0 = ld0.next_step()
    x1, y1 = ld1.next_step()
    l0, l1 = float(tr0.train_step(x0.long(), y0)), float(tr1.train_step(x1.long(), y1))
    assert abs(l0 - l1) < 1e-5                               # zero tables: the first forward is the table-free model
    assert tr1.tables.stats["updates"] == 2 and tr1.tables.stats["touched"] > 0
    assert float(tr1.tables.shards[0].abs().sum()) > 0       # rows moved
    state = tr1.tables.state_for_checkpoint(quantize=True)
    assert state["table_2"].dtype == torch.int8 and state["table_2_scale"].dtype == torch.bfloat16


def test_attention_free_blocks_with_shift_mixer():
    """Round-1 style stack: attention only in some blocks, the others add a learned multiple of the one-token shift."""
    from them_bones_b200.utils.evalbpb import causality_check
    cfg = tiny_cfg(n_layer=4, attn_layers=(0, 2), mixer="shift1", mlp_ratio=6)
    assert model_config_dict(cfg)["attn_layers"] == [0, 2] and GPTConfig(**model_config_dict(cfg)) == cfg
    tr, losses = run_steps(cfg, "lean", steps=8)
    assert losses[-1] < losses[0]
    names = dict(tr.model.named_parameters())
    assert "transformer.h.1.mix_lambda" in names and "transformer.h.1.attn.c_q.weight" not in names
    assert "transformer.h.0.attn.c_q.weight" in names and "transformer.h.0.mix_lambda" not in names
    assert names["transformer.h.1.mlp.c_fc.weight"].shape == (6 * 256, 256)
    assert float(names["transformer.h.1.mix_lambda"].abs().sum()) > 0          # the mixer gain was trained
    x = torch.arange(12.0).view(1, 4, 3)
    assert torch.equal(RF.shift1(x)[0, 1:], x[0, :-1]) and float(RF.shift1(x)[0, 0].abs().sum()) == 0
    assert causality_check(tr.model, 8192, 2, 64, "cpu")["passed"]


def test_multi_token_prediction_targets_and_schedule():
    from them_bones_b200.optim.schedules import mtp_weights
    # the reference's two-target schedule: t+3 fades over the first quarter, t+2 over the second
    assert mtp_weights(0.0, 2) == (0.5, 0.25)
    assert mtp_weights(0.125, 2) == pytest.approx((0.5, 0.125))
    assert mtp_weights(0.375, 2) == pytest.approx((0.25, 0.0))
    assert mtp_weights(0.5, 2) == (0.0, 0.0) and mtp_weights(0.9, 2) == (0.0, 0.0)
    torch.manual_seed(0)
    cfg = tiny_cfg(n_layer=2, mtp_offsets=(2, 3))
    model = GPT(cfg)
    model.init_weights()
    with torch.no_grad():
        model.lm_head.weight.normal_(0, 0.05)
    model.train()
    x = torch.randint(1, 8192, (2, 64))
    x[:, 0] = 0
    x[0, 40] = 0
    y = torch.roll(x, -1, 1)
    y[:, -1] = -1
    y[y == 0] = -1                                             # targets that are a document start are not predicted
    model.set_mtp_weights((0.0, 0.0))
    base = float(model(x, y))
    model.set_mtp_weights((0.5, 0.25))
    terms = model.mtp_terms(y)
    assert len(terms) == 2
    t2, w2 = terms[0]
    assert torch.equal(t2[0, :10], y[0, 1:11]) and int(t2[0, -1]) == -1
    assert float(w2[0, 38]) == 0.0 and float(w2[0, 39]) == 0.0    # y[0, 39] is masked: nothing is predicted across it
    assert float(w2[0, 10]) > 0
    with torch.no_grad():
        h = model.trunk(x)
        manual = base
        for tk, wk in terms:
            manual += float(RF.softcap_cross_entropy(h, model.lm_head.weight, tk, cfg.vocab_size, cfg.softcap, wk))
    full = model(x, y)
    assert float(full) == pytest.approx(manual, rel=1e-5) and float(full) > base
    full.backward()
    assert model.lm_head.weight.grad is not None
    model.eval()
    assert float(model(x, y)) == pytest.approx(base, rel=1e-6)   # evaluation is next-token only


def test_label_smoothing_only_in_training():
    torch.manual_seed(0)
    cfg = tiny_cfg(n_layer=2, label_smoothing=0.1)
    model = GPT(cfg)
    model.init_weights()
    with torch.no_grad():
        model.lm_head.weight.normal_(0, 0.05)
    x = torch.randint(1, 8192, (2, 64))
    y = torch.roll(x, -1, 1)
    model.train()
    smooth = float(model(x, y))
    model.eval()
    plain = float(model(x, y))
    with torch.no_grad():
        h = model.trunk(x)
        want = float(RF.softcap_cross_entropy(h, model.lm_head.weight, y, cfg.vocab_size, cfg.softcap, label_smoothing=0.1))
    assert smooth == pytest.approx(want, rel=1e-6) and smooth != pytest.approx(plain, rel=1e-4)


def test_output_table_keys_signs_and_row_step():
    x = torch.randint(1, 512, (2, 40))
    x[0, 20] = 0                                                              # a BOS inside the first window
    row, hs = RF.os1_keys(x, 4, 1 << 10, bos_id=0, seed=3)
    assert (row[:, :3] == -1).all() and (row[1, 3:] >= 0).all() and int(row.max()) < (1 << 10)
    # a key spans a BOS only as its first id: the keys ending at 20..22 hold the BOS after their first id
    assert (row[0, 20:23] == -1).all() and row[0, 19] >= 0 and row[0, 23] >= 0
    # causal and deterministic: a key depends on its own `order` ids only
    x2 = x.clone()
    x2[1, 10] = (x2[1, 10] % 500) + 7
    row2, hs2 = RF.os1_keys(x2, 4, 1 << 10, bos_id=0, seed=3)
    same = torch.ones(40, dtype=torch.bool)
    same[10:14] = False
    assert (row2[1][same] == row[1][same]).all() and (hs2[1][same] == hs[1][same]).all()
    assert (row2[1, 10:14] != row[1, 10:14]).any()
    sg = RF.os1_signs(hs.reshape(-1), 128)
    assert sg.shape == (80, 128) and set(sg.unique().tolist()) == {-1.0, 1.0}
    assert abs(float(sg.mean())) < 0.05                                       # balanced
    assert torch.equal(sg, RF.os1_signs(hs.reshape(-1), 128))
    # the stateless row step: first step is full size whatever the gradient's scale, then the budget binds
    g = torch.randn(5, 128) * 1e-4
    x1 = RF.os1_row_step(torch.zeros(5, 128), g, lr=0.125, eps=1e-12, cap=4.0)
    assert torch.allclose(x1.square().mean(1).sqrt(), torch.full((5,), 0.125), rtol=1e-3)
    xs = x1
    for _ in range(10):
        xs = RF.os1_row_step(xs, g, lr=0.125, eps=1e-12, cap=4.0)
    assert float(xs.square().mean(1).sqrt().max()) <= 0.5 + 1e-5
    zero = RF.os1_row_step(x1, torch.zeros(5, 128), lr=0.125, eps=1e-12, cap=4.0)
    assert torch.equal(zero, x1)                                              # a zero gradient takes no step


def test_output_table_gate_is_causal_and_readout_gradient():
    torch.manual_seed(0)
    b, t, dim, v = 2, 24, 32, 64
    code = RF.os1_codebook(v, dim, 7)
    u = torch.randn(b * t, dim)
    idx = torch.randint(0, v, (b, t))
    g = RF.os1_gate(u, code, idx, a0=1.0, width=4, h0=0.3, slope=30.0)
    assert g.shape == (b, t) and float(g[0, 0]) == pytest.approx(torch.sigmoid(torch.tensor(-9.0)).item(), rel=1e-5)
    u2, idx2 = u.clone(), idx.clone()
    u2.view(b, t, dim)[:, 12:] += 1.0                                          # later reads ...
    idx2[:, 14:] = (idx2[:, 14:] + 1) % v                                      # ... and later tokens
    g2 = RF.os1_gate(u2, code, idx2, a0=1.0, width=4, h0=0.3, slope=30.0)
    assert torch.equal(g[:, :13], g2[:, :13])                                  # position t reads j <= t-1 and tokens <= t
    # manual value at t = 5: mean over j = 1..4 of u_j . C[idx[j+1]]
    want = torch.stack([(u.view(b, t, dim)[0, j] * code[idx[0, j + 1]]).sum() for j in range(1, 5)]).mean()
    assert float(g[0, 5]) == pytest.approx(torch.sigmoid(30.0 * (want - 0.3)).item(), abs=1e-5)
    # gradient reaches u through the linear term only: du = (glin / a0) * dpre @ C
    x = torch.randn(b * t, 16)
    w = torch.randn(v, 16) * 0.1
    tg = torch.randint(0, v, (b * t,))
    uu = (u * 0.5).requires_grad_(True)
    loss = RF.softcap_cross_entropy_os1(x, w, tg, v, 15.0, uu, code, g.reshape(-1), a0=1.0, glin=0.01, beta=3.0, thr=0.7)
    loss.backward()
    pre = (x @ w.T + RF.os1_readout((uu.detach() @ code.T), g.reshape(-1), 0.01, 3.0, 0.7)).requires_grad_(True)
    torch.nn.functional.cross_entropy(15.0 * torch.tanh(pre / 15.0), tg).backward()
    assert torch.allclose(uu.grad, 0.01 * pre.grad @ code, atol=1e-7)


def test_output_table_zero_init_is_identity_then_learns(tmp_path):
    from them_bones_b200.utils import ckpt as CK
    kw = dict(n_layer=1, n_embd=64, n_head=2, vocab_size=512, sequence_len=64)
    cfg0 = tiny_cfg(**kw)
    cfg1 = tiny_cfg(os1_rows=1 << 12, os1_order=3, os1_dim=32, **kw)
    hy = Hyper()
    hy.total_batch, hy.device_batch = 4 * 64, 2                               # two micro-steps per step
    tr0 = Trainer(cfg0, hy, RT, optimizer_kind="lean", horizon_steps=10)
    tr1 = Trainer(cfg1, hy, RT, optimizer_kind="lean", horizon_steps=10)
    ld = SynthLoader(512, 64, 4, seed=0, doc_len=(16, 64))
    x, y = ld.next_step()
    l0, l1 = float(tr0.train_step(x.long(), y)), float(tr1.train_step(x.long(), y))
    assert abs(l0 - l1) < 1e-5                                # zero rows: the first forward is the table-free model
    st = tr1.os1.stats
    assert st["updates"] == 1 and st["touched"] > 0
    rms = tr1.os1.shard.float().square().mean(1).sqrt()
    moved = rms > 0
    assert st["touched"] - 8 <= int(moved.sum()) <= st["touched"]      # a row read only at masked targets has no gradient
    assert torch.allclose(rms[moved], torch.full_like(rms[moved], cfg1.os1_lr), rtol=1e-3)   # full-size first step
    # the same windows again: rows that were stepped now pull their contexts' next tokens up, beyond what the dense
    # weights' own step gives
    for _ in range(6):
        l0, l1 = float(tr0.train_step(x.long(), y)), float(tr1.train_step(x.long(), y))
    assert l1 < l0 - 0.02, (l0, l1)
    assert float(tr1.os1.shard.float().square().mean(1).sqrt().max()) <= cfg1.os1_lr * hy.os1_cap * 1.001
    # checkpoint: int8 rows + bf16 scales in model_state, the read-out's settings in model_config
    path = str(tmp_path / "os1.pt")
    CK.save_checkpoint(path, tr1.model, dict(steps=7))
    raw = torch.load(path, weights_only=True)
    assert raw["model_state"]["os1_table"].dtype == torch.int8 and raw["model_state"]["os1_scale"].dtype == torch.bfloat16
    assert raw["model_config"]["os1_rows"] == 1 << 12 and raw["model_config"]["os1_order"] == 3
    model, _ = CK.load_for_eval(path, "cpu")
    xe = x[:2].long()
    with torch.no_grad():
        tr1.model.eval()
        a, bb = model(xe), tr1.model(xe)
        tr1.model.train()
    # int8 rows: a score just above the threshold moves by the quantisation step times the thresholded term's gain
    assert float((a - bb).abs().mean()) < 2e-3 and float((a - bb).abs().max()) < 0.5
    assert model(xe, y[:2], loss_reduction="none").shape == (2, 64)


def test_answer_span_marks_and_weighted_loss():
    import numpy as np
    from them_bones_b200.data.synth import slice_windows, tail_marks
    row = np.array([0, 5, 6, 7, 8, 9, 10, 11, 0, 3, 4, 5, 0, 9, 9, 9, 9], dtype=np.int32)      # docs of 8, 4 and 5 tokens
    m = tail_marks(row, 0, 0.25)
    assert m.tolist() == [False] * 6 + [True] * 2 + [False] * 3 + [True] + [False] * 4 + [True]
    x, y = slice_windows(row, 8, 0, mark_tail=0.25, vocab=100)
    assert x.shape == (2, 8) and y.shape == (2, 8)
    assert y[0].tolist() == [5, 6, 7, 8, 9, 110, 111, -1]               # marked targets carry +vocab; BOS stays masked
    assert y[1].tolist() == [3, 4, 105, -1, 9, 9, 9, 109]
    x0, y0 = slice_windows(row, 8, 0)
    assert (np.where(y >= 100, y - 100, y) == y0).all()
    # the model unmarks and weights: loss = sum(w * nll) / count(valid)
    torch.manual_seed(0)
    cfg = tiny_cfg(n_layer=1, n_embd=64, n_head=2, vocab_size=512, sequence_len=32)
    model = GPT(cfg)
    model.init_weights()
    with torch.no_grad():
        model.lm_head.weight.normal_(0, 0.05)
    idx = torch.randint(1, 512, (2, 32))
    tg = torch.randint(1, 512, (2, 32))
    tg[0, 5] = -1
    marked = torch.zeros(2, 32, dtype=torch.bool)
    marked[:, 24:] = True
    tgm = torch.where(marked & (tg >= 0), tg + 512, tg)
    model.answer_weight = 3.0
    model.train()
    got = model(idx, tgm, loss_div=2.0)
    nll = model(idx, tg, loss_reduction="none")
    w = torch.where(marked, 3.0, 1.0) * (tg >= 0)
    assert float(got) == pytest.approx(float((w * nll).sum() / (tg >= 0).sum() / 2.0), rel=1e-5)
    model.eval()
    assert torch.allclose(model(idx, tgm, loss_reduction="none"), nll)     # evaluation unmarks, no weights
    model.answer_weight = None
    model.train()
    assert float(model(idx, tg, loss_div=2.0)) == pytest.approx(float(nll.sum() / (tg >= 0).sum() / 2.0), rel=1e-5)


def test_split_evaluation_classes_and_totals():
    import numpy as np
    from them_bones_b200.utils.evalbpb import evaluate_bpb
    from them_bones_b200.utils.evalsplit import ContextSet, SplitEval, bigram_repeats, evaluate_split
    x = np.array([[0, 5, 6, 5, 6, 0, 5, 6]])
    y = np.array([[5, 6, 5, 6, -1, 5, 6, 7]])
    rep = bigram_repeats(x, y, 0)
    assert rep.tolist() == [[False, False, False, True, False, False, False, False]]     # (5,6) again in document 1 only
    cs = ContextSet(ctx=2)
    cs.add(np.array([9, 5, 6, 9]))
    seen = cs.seen(x)
    assert seen.tolist() == [[False, False, True, False, True, False, False, True]]      # context (5,6) ends at 2, 4, 7
    ev = SplitEval(16, 0, cs, token_bytes=torch.full((16,), 2))
    ev.observe(torch.from_numpy(x), torch.from_numpy(y), torch.ones(1, 8))
    m = ev.merged()
    assert m["all"]["tokens"] == 7 and m["bi_rep"]["tokens"] == 1 and m["ctx_seen"]["tokens"] == 2
    assert m["novel"]["tokens"] == 4 and m["all"]["bytes"] == 14 and m["all"]["nats"] == pytest.approx(7.0)
    # on a model: the "all" class is evaluate_bpb's number
    torch.manual_seed(0)
    model = GPT(tiny_cfg(n_layer=1, n_embd=64, n_head=2, vocab_size=512, sequence_len=64))
    model.init_weights()
    a = evaluate_bpb(model, 512, 4, 64, torch.device("cpu"), max_tokens=1000)
    b = evaluate_split(model, 512, 4, 64, torch.device("cpu"), max_tokens=1000)
    assert b["all"]["bpb"] == pytest.approx(a["val_bpb"], rel=1e-6) and b["all"]["tokens"] == a["num_tokens"]
    assert b["bi_rep"]["tokens"] + b["novel"]["tokens"] == b["all"]["tokens"]


def test_background_checkpoint_write(tmp_path):
    from them_bones_b200.utils import ckpt as CK
    model = GPT(tiny_cfg(n_layer=1, n_embd=64, n_head=2, vocab_size=512, sequence_len=64))
    model.init_weights()
    bg = CK.BackgroundSave()
    for k in range(2):                                           # the second submit waits for the first
        bg.submit(str(tmp_path / f"p{k}.pt"), CK.build_payload(model, dict(steps=k)))
    bg.wait()
    assert bg.done == 2
    m, meta = CK.load_for_eval(str(tmp_path / "p1.pt"), "cpu")
    assert meta["steps"] == 1 and torch.equal(m.lm_head.weight, model.lm_head.weight)
    CK.check_declared_length(model, 64)
    with pytest.raises(RuntimeError):
        CK.check_declared_length(model, 32)
    bg.submit(str(tmp_path / "no_such_dir" / "x" / ".." / ".." / "f\0.pt"), dict(a=1))
    with pytest.raises(RuntimeError):
        bg.wait()


@pytest.mark.parametrize("bits", [1, 4])
def test_packed_table_views_train_straight_through_and_round_trip(tmp_path, bits):
    from them_bones_b200.utils import ckpt as CK
    m = torch.randn(5, 32) * 0.3
    m[1] = 0
    v = RF.table_view(m, bits)
    assert float(v[1].abs().sum()) == 0 and torch.equal(RF.table_view(v, bits), v)          # zero stays zero; idempotent
    if bits == 1:
        assert torch.allclose(v.abs()[0], m[0].abs().mean().bfloat16().float().expand(32)) and torch.equal(v.sign()[0], torch.where(m[0] < 0, -1.0, 1.0))
    else:
        assert float((v - m).abs().max()) <= float(m.abs().amax()) / 7 * 0.51 + 1e-3 and len(torch.unique(v[0])) <= 15
    pk, sc = RF.table_pack_view(m, bits)
    assert pk.dtype == torch.uint8 and pk.shape == (5, 32 * bits // 8) and sc.dtype == torch.bfloat16
    assert torch.allclose(RF.table_unpack_view(pk, sc, bits), v, atol=1e-6)
    # both kinds of table read their views in training, learn through them, and save them packed
    kw = dict(n_layer=1, n_embd=64, n_head=2, vocab_size=512, sequence_len=64)
    cfg = tiny_cfg(table_orders=(2,), table_rows=1 << 10, table_bits=bits, os1_rows=1 << 10, os1_order=2, os1_dim=32,
                   os1_bits=1, **kw)
    hy = Hyper()
    hy.total_batch, hy.device_batch = 4 * 64, 4
    tr = Trainer(cfg, hy, RT, optimizer_kind="lean", horizon_steps=10)
    x, y = SynthLoader(512, 64, 4, seed=0, doc_len=(16, 64)).next_step()
    losses = [float(tr.train_step(x.long(), y)) for _ in range(6)]
    assert losses[-1] < losses[0] - 0.5
    assert float(tr.tables.shards[0].abs().sum()) > 0 and float(tr.os1.shard.abs().sum()) > 0
    path = str(tmp_path / "views.pt")
    CK.save_checkpoint(path, tr.model, dict(steps=6), tables=tr.tables)
    raw = torch.load(path, weights_only=True)["model_state"]
    assert raw["table_2"].dtype == torch.uint8 and raw["table_2"].shape == (1 << 10, 64 * bits // 8)
    assert raw["os1_table"].dtype == torch.uint8 and raw["os1_table"].shape == (1 << 10, 4)
    model, _ = CK.load_for_eval(path, "cpu")
    assert model.tables.rows_are_views and model.os1.rows_are_views
    tr.model.eval()
    with torch.no_grad():
        a, b = model(x[:2].long()), tr.model(x[:2].long())
    assert torch.allclose(a, b, atol=2e-4)                        # the scored forward is the trained forward


def test_grad_clip_and_bf16_stochastic_masters(monkeypatch):
    from them_bones_b200 import config as C
    # stochastic rounding is unbiased and lands on the two neighbouring bf16 values
    x = torch.full((200000,), 1.0 + 2.0 ** -10)
    y = RF.stochastic_round_bf16(x, torch.Generator().manual_seed(0)).float()
    assert set(y.unique().tolist()) == {1.0, 1.0 + 2.0 ** -7} and abs(float(y.mean()) - float(x[0])) < 2e-5
    assert torch.equal(RF.stochastic_round_bf16(torch.tensor([0.5, -2.0, float("inf")])).float(), torch.tensor([0.5, -2.0, float("inf")]))
    cfg = tiny_cfg(n_layer=2, n_embd=64, n_head=2, vocab_size=512, sequence_len=64)
    base = run_steps(cfg, "lean", steps=6, seq=64, batch=4)[1]
    monkeypatch.setenv("BONES_GRAD_CLIP", "0.05")
    C.switches(refresh=True)
    tr, clipped = run_steps(cfg, "lean", steps=6, seq=64, batch=4)
    assert float(tr.optimizer.last_grad_norm) > 0.05                      # the clip was active ...
    assert clipped[0] == pytest.approx(base[0], abs=1e-5) and clipped[-1] < clipped[0]
    assert any(abs(a - b) > 1e-4 for a, b in zip(base[1:], clipped[1:]))      # ... and changed the AdamW groups' steps
    monkeypatch.delenv("BONES_GRAD_CLIP")
    monkeypatch.setenv("BONES_MASTER", "bf16")
    C.switches(refresh=True)
    tr, lossy = run_steps(cfg, "lean", steps=6, seq=64, batch=4)
    assert tr.optimizer.muon_units[0].master.dtype == torch.bfloat16
    assert all(abs(a - b) < 0.05 for a, b in zip(base, lossy)) and lossy[-1] < lossy[0] - 0.1
    monkeypatch.delenv("BONES_MASTER")
    C.switches(refresh=True)


def test_cached_decode_with_moe_blocks_and_tables_matches_full_recompute():
    """The KV-cache route carries the token history for the table hashes and routes one token per sequence through the
    experts; it must reproduce the cache-free route token for token."""
    from them_bones_b200.models.tables import HashedTables
    from them_bones_b200.utils.decode import greedy_decode, greedy_decode_full
    cfg = GPTConfig(sequence_len=256, vocab_size=2048, n_layer=2, n_head=2, n_embd=128, doc_mask=True, moe_layers=(1,),
                    moe_experts=4, moe_topk=2, moe_capacity=40, moe_hidden=128, table_orders=(2, 3), table_rows=1 << 10)
    torch.manual_seed(0)
    m = GPT(cfg)
    m.init_weights()
    with torch.no_grad():
        for blk in m.transformer.h:
            blk.attn.c_proj.weight.normal_(0, 0.05)
        m.transformer.h[0].mlp.c_proj.weight.normal_(0, 0.05)
        m.transformer.h[1].mlp.w_proj.normal_(0, 0.05)
        m.lm_head.weight.normal_(0, 0.3)
    t = HashedTables(cfg.table_orders, cfg.table_rows, cfg.n_embd)
    for sh in t.shards:
        sh.copy_(torch.randn_like(sh) * 0.3)
    m.attach_tables(t)
    m.eval()
    pr = torch.randint(1, 2048, (3, 20))
    pr[:, 0] = 0
    pr[1, 10] = 0
    assert torch.equal(greedy_decode(m, pr, 10), greedy_decode_full(m, pr, 10))
