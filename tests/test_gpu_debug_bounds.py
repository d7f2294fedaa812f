"""The bounds-checked library build (``-DBONES_DEBUG_BOUNDS``): a clean MoE + tables training step trips no check, and an
index that lies outside its extent is counted with its value and skipped instead of being dereferenced.  Run in a child
process because the choice of library is made when ``ops._lib`` is first imported."""
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

CHILD = r'''
import ctypes, torch
from them_bones_b200.ops import _lib as L
assert L.DEBUG_BOUNDS and L.lib_path().endswith("_dbg.so")
from them_bones_b200.config import GPTConfig, Hyper
from them_bones_b200.data.synth import SynthLoader
from them_bones_b200.runtime import Runtime
from them_bones_b200.trainer import Trainer
rt = Runtime(False, 0, 0, 1, torch.device("cuda", 0), "cuda")
cfg = GPTConfig(sequence_len=256, vocab_size=2048, n_layer=2, n_head=2, n_embd=256, head_dim=128, doc_mask=True,
                moe_layers=(1,), moe_experts=4, moe_topk=2, moe_capacity=40, moe_hidden=256, table_orders=(2, 3), table_rows=1 << 12)
hy = Hyper(); hy.total_batch, hy.device_batch = 4 * 256, 4
tr = Trainer(cfg, hy, rt, horizon_steps=10)
ld = SynthLoader(cfg.vocab_size, 256, tr.local_windows, seed=0, doc_len=(32, 256), pin=True)
for _ in range(2):
    tr.train_step(*ld.next_step())
torch.cuda.synchronize()
tr.check_device_health()                       # error word, canaries and the bounds counters: all clean
assert L.bounds_hits() == {}
# an embedding gather with one id beyond the table: caught, counted, skipped (the row comes back as zeros)
table = torch.randn(100, 64, device="cuda").bfloat16()
idx = torch.tensor([3, 250, 7], device="cuda")
out = torch.full((3, 64), 9.0, device="cuda").bfloat16()
L.call("bones_gather_rows", L.ptr(table), L.ptr(idx), ctypes.c_int(1), L.ptr(out), ctypes.c_int(3), ctypes.c_int(64),
       ctypes.c_longlong(100), L.stream())
torch.cuda.synchronize()
hits = L.bounds_hits()
assert hits["elementwise"][0] >= 1 and hits["elementwise"][1] == 250, hits      # every lane of the row's warp reports it
assert torch.equal(out[0], table[3]) and float(out[1].float().abs().sum()) == 0.0
assert L.bounds_hits() == {}                   # read and cleared
print("DEBUG_BOUNDS_OK")
'''


def test_debug_bounds_build_is_clean_on_a_training_step_and_catches_a_bad_index():
    env = dict(os.environ, PYTHONPATH=ROOT, BONES_DEBUG_BOUNDS="1")
    out = subprocess.run([sys.executable, "-c", CHILD], env=env, cwd=ROOT, capture_output=True, text=True, timeout=600)
    assert out.returncode == 0 and "DEBUG_BOUNDS_OK" in out.stdout, out.stdout[-1500:] + out.stderr[-3000:]
