"""Expert parallelism on real GPUs (needs >= 2 B200 on the box, else skipped): both transports against the
single-GPU fused layer, eager and replayed from a CUDA graph (tests/multi/ep_worker.py), and continuous
batching through B200Backend with different requests on every rank (tests/multi/ep_backend_worker.py), each
under torchrun.  NVLS is switched off for these child processes: the ranks exchange by plain peer stores."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_both_transports_match_the_fused_layer_on_two_gpus():
    worker = os.path.join(os.path.dirname(os.path.abspath(__file__)), "multi", "ep_worker.py")
    n = 2
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}",
           "--master-addr", "127.0.0.1", "--master-port", "29533", worker]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=240, env=dict(os.environ, NCCL_NVLS_ENABLE="0"))
    tail = (r.stdout + r.stderr)[-3000:]
    assert r.returncode == 0, tail
    for rank in range(n):
        assert f"EP_MULTI_OK {rank}" in r.stdout, tail


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_continuous_batching_with_different_requests_per_rank_matches_a_single_gpu_engine():
    worker = os.path.join(os.path.dirname(os.path.abspath(__file__)), "multi", "ep_backend_worker.py")
    n = 2
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}",
           "--master-addr", "127.0.0.1", "--master-port", "29534", worker]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=300, env=dict(os.environ, NCCL_NVLS_ENABLE="0"))
    tail = (r.stdout + r.stderr)[-4000:]
    assert r.returncode == 0, tail
    for rank in range(n):
        assert f"EP_BACKEND_OK {rank}" in r.stdout, tail
