"""CPU tests of the resume path (model state + per-rank optimizer state), the agreed training clock and the tail-average
save (the checkpoint must equal the model that was evaluated)."""
import torch

from them_bones_b200.config import GPTConfig, Hyper
from them_bones_b200.data.synth import SynthLoader
from them_bones_b200.runtime import Runtime
from them_bones_b200.trainer import Trainer
from them_bones_b200.utils import ckpt as CK

RT = Runtime(False, 0, 0, 1, torch.device("cpu"), "cpu")


def _cfg():
    return GPTConfig(sequence_len=128, vocab_size=2048, n_layer=2, n_head=2, n_embd=128, rope_base=10000.0, doc_mask=True)


def _trainer(init_state=None):
    h = Hyper()
    h.total_batch, h.device_batch = 4 * 128, 4
    return Trainer(_cfg(), h, RT, optimizer_kind="lean", horizon_steps=20, init_state=init_state)


def test_resume_continues_bit_for_bit(tmp_path):
    ld = SynthLoader(2048, 128, 4, seed=1, doc_len=(32, 128))
    batches = [ld.next_step() for _ in range(5)]
    tr = _trainer()
    for x, y in batches[:3]:
        tr.train_step(x.long(), y)
    path = str(tmp_path / "mid.pt")
    CK.save_checkpoint(path, tr.model, dict(steps=3), optimizer=tr.optimizer)
    assert CK.save_optimizer_state(path, tr.optimizer, 0) == path + ".opt.rank0"
    want = [float(tr.train_step(x.long(), y)) for x, y in batches[3:]]

    ck = torch.load(path, weights_only=True)
    tr2 = _trainer(init_state=ck["model_state"])
    tr2.optimizer.load_unit_state_dict(torch.load(CK.opt_state_path(path, 0), weights_only=True))
    tr2.step_index = 3
    got = [float(tr2.train_step(x.long(), y)) for x, y in batches[3:]]
    assert got == want

    # without the optimizer state the weights still load, but the momentum is gone: the second resumed step differs
    tr3 = _trainer(init_state=ck["model_state"])
    tr3.step_index = 3
    cold = [float(tr3.train_step(x.long(), y)) for x, y in batches[3:]]
    assert cold[0] == want[0] and cold[1] != want[1]


def test_optimizer_state_refuses_another_rank_layout():
    tr = _trainer()
    sd = tr.optimizer.unit_state_dict()
    sd["world"] = 2
    try:
        tr.optimizer.load_unit_state_dict(sd)
    except ValueError:
        return
    raise AssertionError("a two-rank state loaded into a one-rank optimizer")


def test_progress_follows_the_agreed_clock():
    h = Hyper()
    h.total_batch, h.device_batch = 4 * 128, 4
    tr = Trainer(_cfg(), h, RT, optimizer_kind="lean", budget_seconds=100.0)
    tr.t_start -= 50.0                               # this rank's own clock says half way
    assert 0.45 < tr.progress() < 0.6
    tr.set_agreed_clock(10.0)                        # rank 0 says a tenth: that is what every rank uses
    assert tr.progress() == 0.1
    tr.set_agreed_clock(1000.0)
    assert tr.progress() == 1.0


def test_tail_average_checkpoint_equals_the_evaluated_model(tmp_path):
    from them_bones_b200.utils.ema import EmaLawa
    ld = SynthLoader(2048, 128, 4, seed=2, doc_len=(32, 128))
    tr = _trainer()
    ema = EmaLawa(tr.model.parameters(), 0.0, 1)
    for step in range(3):
        x, y = ld.next_step()
        tr.train_step(x.long(), y)
        ema.update(step, 1.0)
    ema.swap_in()
    path = str(tmp_path / "final.pt")
    CK.save_checkpoint(path, tr.model, dict(steps=3), optimizer=None)      # what train.py does after a swap-in
    state = torch.load(path, weights_only=True)["model_state"]
    for name, p in tr.model.named_parameters():
        assert torch.equal(state[name], p.detach()), name
    # the owners' masters still hold the un-averaged weights: saving through the optimizer would not be the same model
    masters = tr.optimizer.consolidated_state_dict()
    assert any(not torch.equal(masters[p], p.detach().float()) for p in masters)


def test_health_check_counts_non_finite_steps():
    tr = _trainer()
    ld = SynthLoader(2048, 128, 4, seed=3, doc_len=(32, 128))
    x, y = ld.next_step()
    tr.train_step(x.long(), y)
    assert tr.check_device_health() == 0
    opt = tr.optimizer
    opt.zero_grad()
    opt.muon_units[0].G.fill_(float("nan"))          # a poisoned gradient: the gate zeroes the step's gradients
    opt.step()
    assert tr.check_device_health() == 1
    for n, p in tr.model.named_parameters():
        assert torch.isfinite(p).all(), n
