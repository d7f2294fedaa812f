"""Stand-in for the competition kit module ``prepare`` that the reference programs import but do not ship
(``from prepare import ...`` at round2/source/train.py:59-73).  It supplies the thirteen names with synthetic data of
the benchmark's shape, so the *unmodified* reference ``train.py`` can run: Zipf(1.1) token ids, documents of 128-2048
tokens starting with BOS, best-fit packed rows, ``inputs = row[:-1]`` (int32) and ``targets = row[1:]`` (int64), the same
stream the framework's own loader produces.

``record_step_boundary`` keeps a wall-clock stamp per optimizer step; the reference calls it right after its own
``synchronize()``, so differences of consecutive stamps are device-complete step times.  The stamps are written to the
file named by ``BONES_REF_STAMPS`` when the process exits.
"""
import atexit
import json
import os
import sys
import time

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from them_bones_b200.data.synth import PackedRows, ZipfDocs, bytes_per_token_table  # noqa: E402

TOKENIZER_VOCAB_SIZE = int(os.environ.get("BONES_REF_VOCAB", 65536))
TRAIN_TIME_BUDGET_SECONDS = int(os.environ.get("BONES_REF_BUDGET", 4 * 3600))
TRAIN_STARTUP_STEPS_EXCLUDED = 5
TRAIN_STARTUP_ALLOWANCE_CAP_SECONDS = 3600
EVAL_TIMEOUT_SECONDS = 600
_BOS = 0
_STAMPS = []


def get_dist_info():
    if "RANK" in os.environ and "WORLD_SIZE" in os.environ:
        return True, int(os.environ["RANK"]), int(os.environ.get("LOCAL_RANK", 0)), int(os.environ["WORLD_SIZE"])
    return False, 0, 0, 1


def print0(*args, **kw):
    if int(os.environ.get("RANK", 0)) == 0:
        print(*args, **kw, flush=True)


class Tokenizer:
    """Synthetic tokenizer: ids are already tokens; ``encode`` maps text to deterministic ids for API completeness."""
    enc = None

    def get_bos_token_id(self):
        return _BOS

    def get_vocab_size(self):
        return TOKENIZER_VOCAB_SIZE

    def encode(self, texts, prepend=None, num_threads=1):
        out = []
        for t in texts:
            ids = [1 + (hash(w) % (TOKENIZER_VOCAB_SIZE - 1)) for w in str(t).split()]
            out.append(([prepend] if prepend is not None else []) + ids)
        return out


def ensure_tokenizer(build_if_missing=False):
    return Tokenizer()


def make_dataloader(tokenizer, batch, seq_len, split, device):
    """Generator of ``(inputs int32 [batch, seq_len], targets int64 [batch, seq_len], {"epoch": n})``."""
    _, rank, _, _ = get_dist_info()
    seed = (1234 if split == "train" else 4321) * 1000003 + rank
    docs = ZipfDocs(TOKENIZER_VOCAB_SIZE, 1.1, (128, 2048), seed=seed, bos_id=_BOS)
    rows = PackedRows(docs, seq_len)
    dev = torch.device(device) if not isinstance(device, torch.device) else device
    pin = dev.type == "cuda"
    while True:
        buf = torch.empty(batch, seq_len + 1, dtype=torch.int32)
        for i in range(batch):
            buf[i] = torch.from_numpy(rows.next_row())
        if pin:
            buf = buf.pin_memory()
        x = buf[:, :-1].to(dev, non_blocking=True).contiguous()
        y = buf[:, 1:].to(dev, non_blocking=True).to(torch.int64).contiguous()
        yield x, y, {"epoch": 1}


def record_step_boundary(step):
    _STAMPS.append((int(step), time.perf_counter()))


@atexit.register
def _dump_stamps():
    path = os.environ.get("BONES_REF_STAMPS")
    if path and int(os.environ.get("RANK", 0)) == 0:
        with open(path, "w") as fh:
            json.dump(_STAMPS, fh)


@torch.no_grad()
def causality_check(model, tokenizer, batch, seq_len, device):
    x = torch.randint(1, TOKENIZER_VOCAB_SIZE, (batch, seq_len), device=device)
    x2 = x.clone()
    cut = seq_len // 2
    x2[:, cut:] = torch.randint(1, TOKENIZER_VOCAB_SIZE, (batch, seq_len - cut), device=device)
    a, b = model(x).float(), model(x2).float()
    diff = float((a[:, :cut] - b[:, :cut]).abs().max())
    return {"passed": diff < 5e-2, "max_abs_diff": diff}


@torch.no_grad()
def evaluate_bpb(model, tokenizer, batch, seq_len, device, split="public_val", max_tokens=1 << 20, timeout_seconds=600):
    import math
    t0 = time.time()
    nbytes = bytes_per_token_table(TOKENIZER_VOCAB_SIZE).to(device)
    loader = make_dataloader(tokenizer, batch, seq_len, split, device)
    nats, nb, ntok = 0.0, 0, 0
    while ntok < max_tokens and time.time() - t0 < timeout_seconds:
        x, y, _ = next(loader)
        loss = model(x, y, loss_reduction="none")
        valid = y != _BOS
        nats += float((loss * valid).sum())
        nb += int((nbytes[y] * valid).sum())
        ntok += int(valid.sum())
    return {"val_bpb": nats / (math.log(2) * max(nb, 1)), "eval_seconds": time.time() - t0, "num_tokens": ntok,
            "eval_timeout": timeout_seconds, "eval_over_timeout": time.time() - t0 > timeout_seconds}
