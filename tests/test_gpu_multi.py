"""Multi-GPU tests (skipped with fewer than two devices): run workers under torch.distributed.run."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _run(worker: str, nproc: int, timeout: int = 600, port: int = 29541):
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}",
           "--master-addr", "127.0.0.1", "--master-port", str(port), os.path.join(ROOT, "tests", "workers", worker)]
    return subprocess.run(cmd, env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, timeout=timeout)


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs >= 2 GPUs")
def test_fused_dp_matches_nccl_baseline():
    n = min(torch.cuda.device_count(), 4)
    r = _run("dp_worker.py", n)
    assert r.returncode == 0 and "DP_WORKER_OK" in r.stdout, r.stdout[-4000:]


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs >= 2 GPUs")
def test_fused_tensor_parallel_kernels():
    n = 4 if torch.cuda.device_count() >= 4 else 2
    r = _run("tp_worker.py", n, port=29543)
    assert r.returncode == 0 and "TP_WORKER_OK" in r.stdout, r.stdout[-4000:]


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs >= 2 GPUs")
def test_fused_expert_parallel_moe():
    n = 4 if torch.cuda.device_count() >= 4 else 2
    r = _run("ep_worker.py", n, port=29545)
    assert r.returncode == 0 and "EP_WORKER_OK" in r.stdout, r.stdout[-4000:]


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs >= 2 GPUs")
def test_fused_ring_attention():
    n = 4 if torch.cuda.device_count() >= 4 else 2
    r = _run("cp_worker.py", n, port=29547)
    assert r.returncode == 0 and "CP_WORKER_OK" in r.stdout, r.stdout[-4000:]


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs >= 2 GPUs")
def test_tensor_and_expert_parallel_serving_slices():
    n = 4 if torch.cuda.device_count() >= 4 else 2
    r = _run("tp_serve_gpu_worker.py", n, port=29549)
    assert r.returncode == 0 and "TP_SERVE_GPU_WORKER_OK" in r.stdout, r.stdout[-4000:]


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs >= 2 GPUs")
def test_pretrain_native_kernels_and_identical_replicas():
    r = _run("pretrain_dp_worker.py", 2, port=29551)
    assert r.returncode == 0 and r.stdout.count("PRETRAIN_DP_WORKER_OK") == 2, r.stdout[-4000:]


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs >= 2 GPUs")
def test_context_parallel_attention_forward_and_backward():
    n = 4 if torch.cuda.device_count() >= 4 else 2
    r = _run("cp_train_worker.py", n, port=29553)
    assert r.returncode == 0 and r.stdout.count("CP_TRAIN_WORKER_OK") == n, r.stdout[-4000:]


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs >= 2 GPUs")
def test_expert_parallel_training_matches_the_unsharded_model():
    """Sharded expert stacks, differentiable all-to-all, grouped tcgen05 GEMMs for the local experts and their gradients."""
    n = 4 if torch.cuda.device_count() >= 4 else 2
    r = _run("ep_train_worker.py", n, port=29555)
    assert r.returncode == 0 and r.stdout.count("EP_TRAIN_WORKER_OK") == n, r.stdout[-4000:]
