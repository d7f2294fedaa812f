"""Scoring / generation entry point (reference: round2/submission/inference.py:18-53).

``load_for_eval(checkpoint_path, device)`` returns a ``ModelWrapper`` whose ``forward(input_ids)`` gives fp32 softcapped
logits ``[B, T, V]``; ``get_eval_worker()`` treats every rank as an independent replica.  Beyond the reference (which
scores full sequences only) the wrapper offers ``score(tokens, ctx_len, total_len)`` (continuation log-likelihoods from a
batched prefill) and ``generate(prompts, n_new)`` (greedy decoding with a KV cache).
"""
from __future__ import annotations

import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

from them_bones_b200.utils import ckpt as CK  # noqa: E402
from them_bones_b200.utils.evalbpb import score_continuations  # noqa: E402
from them_bones_b200.utils.decode import greedy_decode  # noqa: E402


class ModelWrapper(torch.nn.Module):
    def __init__(self, model, meta):
        super().__init__()
        self.model, self.meta = model, meta

    @property
    def config(self):
        return self.model.config

    @torch.no_grad()
    def forward(self, input_ids: torch.Tensor) -> torch.Tensor:
        return self.model(input_ids)

    @torch.no_grad()
    def score(self, tokens, ctx_len, total_len):
        return score_continuations(self.model, tokens, ctx_len, total_len)

    @torch.no_grad()
    def generate(self, prompts: torch.Tensor, n_new: int) -> torch.Tensor:
        return greedy_decode(self.model, prompts, n_new)

    def get_eval_worker(self):
        rank = int(os.environ.get("RANK", 0))
        world = int(os.environ.get("WORLD_SIZE", 1))
        return rank, world


def load_for_eval(checkpoint_path: str, device="cuda", rt=None):
    """``rt``: a multi-rank runtime serves the model sharded (experts and table rows split over the ranks, which then
    score and decode in lockstep); without it every rank is an independent replica, as in the reference."""
    model, meta = CK.load_for_eval(checkpoint_path, device, rt=rt)
    return ModelWrapper(model, meta)


if __name__ == "__main__":
    import argparse
    ap = argparse.ArgumentParser()
    ap.add_argument("checkpoint")
    ap.add_argument("--device", default="cuda" if torch.cuda.is_available() else "cpu")
    ap.add_argument("--new-tokens", type=int, default=16)
    a = ap.parse_args()
    w = load_for_eval(a.checkpoint, a.device)
    cfg = w.model.config
    prompts = torch.randint(1, cfg.vocab_size, (2, 8), device=a.device)
    print(w.generate(prompts, a.new_tokens).tolist())
