"""GPU, two or more devices: the fused sequence-shard exchange (peer loads in the gather, peer stores
in the attention epilogue) gives the same bits as the all-to-all form and as the single-GPU call.
Skipped on a one-GPU box; the host-side shard arithmetic is covered on CPU by test_parallel_gloo.py."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_fused_exchange_matches_all_to_all_and_single_gpu():
    if not torch.cuda.is_available() or torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    out = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2",
                          "--master-addr", "127.0.0.1", "--master-port", "29533",
                          os.path.join(ROOT, "tests", "multi_gpu_worker.py")],
                         capture_output=True, text=True, timeout=600, cwd=ROOT, env=env)
    assert out.returncode == 0 and "MULTI_GPU_OK 2" in out.stdout, (out.stdout[-2000:], out.stderr[-4000:])
