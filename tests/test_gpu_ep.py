"""Expert-parallel layer on 2 GPUs against the single-GPU layer (skipped with fewer than two
devices). Each case is a fresh `torch.distributed.run` job with its own process group, as the
reference's expert-parallel tests are (tests/expert_parallel/_gate.py:19-197)."""

import os
import subprocess
import sys
from pathlib import Path

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent


@pytest.mark.parametrize("expert_map,mode", [("contiguous", "softmax_then_topk"), ("strided", "sigmoid_noaux_tc")])
def test_two_rank_layer_matches_single_gpu(expert_map, mode):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
           "--master-addr", "127.0.0.1", "--master-port", "29613", str(ROOT / "tests" / "ep_worker.py"),
           expert_map, mode]
    done = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env, cwd=str(ROOT))
    assert done.returncode == 0, done.stdout[-3000:] + done.stderr[-3000:]
    assert "ep worker ok" in done.stdout


def test_two_rank_expert_lora_matches_single_gpu():
    """Expert LoRA with a frozen base under expert parallelism against `expert_lora` on one GPU."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
           "--master-addr", "127.0.0.1", "--master-port", "29614", str(ROOT / "tests" / "ep_lora_worker.py")]
    done = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env, cwd=str(ROOT))
    assert done.returncode == 0, done.stdout[-3000:] + done.stderr[-3000:]
    assert "ep lora worker ok" in done.stdout


def test_two_rank_parity_check_with_and_without_presummed_returns():
    """`ep.parity_check` (what bench.py runs before its timed region at N > 1): group-limited
    sigmoid routing with the de-duplicated dispatch, returning one pre-weighted row per token
    copy (within the bf16 tolerance of the single-GPU output) or one row per assignment
    (bit-equal), and plain softmax routing."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
           "--master-addr", "127.0.0.1", "--master-port", "29615", str(ROOT / "tests" / "ep_check_worker.py")]
    done = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env, cwd=str(ROOT))
    assert done.returncode == 0, done.stdout[-3000:] + done.stderr[-3000:]
    assert "ep check worker ok" in done.stdout


def test_two_rank_module_with_autograd():
    """`ExpertParallelLayer`: nn.Module parameters, autograd through `forward`, caller-supplied
    routes, replicated-parameter broadcast and gradient reduction, `close()`."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
           "--master-addr", "127.0.0.1", "--master-port", "29616", str(ROOT / "tests" / "ep_module_worker.py")]
    done = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env, cwd=str(ROOT))
    assert done.returncode == 0, done.stdout[-3000:] + done.stderr[-3000:]
    assert "ep module worker ok" in done.stdout
