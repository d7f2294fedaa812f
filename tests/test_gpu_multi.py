"""Multi-GPU tests (need >= 2 GPUs): fused peer-memory optimizer collectives against the NCCL path."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
@pytest.mark.parametrize("push", ["0", "1"])
def test_fused_optimizer_collectives_match_nccl(push):
    """``push=1``: the weight-gradient GEMMs add their tiles into the owning rank's gradient slab (GEMM -> reduce-scatter
    in one kernel, NVLink atomics from the epilogue); the result must still match the NCCL path."""
    env = dict(os.environ, PYTHONPATH=ROOT, NCCL_NVLS_ENABLE="0", BONES_WGRAD_PUSH=push)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr", "127.0.0.1",
           "--master-port", str(29631 + int(push)), "-m", "them_bones_b200.parallel.selftest"]
    out = subprocess.run(cmd, env=env, cwd=ROOT, capture_output=True, text=True, timeout=600)
    assert out.returncode == 0 and "SELFTEST OK" in out.stdout, out.stdout[-2000:] + out.stderr[-2000:]
