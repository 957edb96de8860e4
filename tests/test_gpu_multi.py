"""Fused layer on 2 (and, when present, 4 or 8) GPUs of one node against the dense oracle, as child processes."""
import os
import signal
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _run(world, port, worker="mgpu_worker.py", token="MGPU_OK", timeout=600, args=()):
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", CCFUSER_WAIT_LIMIT_S="20")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
           "--master-addr", "127.0.0.1", "--master-port", str(port), os.path.join(ROOT, "tests", worker)] + list(args)
    # own session: if the run has to be cut short, the launcher and all its ranks go together
    proc = subprocess.Popen(cmd, env=env, stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True, start_new_session=True)
    try:
        stdout, stderr = proc.communicate(timeout=timeout)
    except subprocess.TimeoutExpired:
        os.killpg(proc.pid, signal.SIGKILL)
        stdout, stderr = proc.communicate()
        raise AssertionError(f"timed out after {timeout} s\n" + stdout[-3000:] + stderr[-3000:])
    assert proc.returncode == 0 and token in stdout, stdout[-3000:] + stderr[-3000:]


@pytest.mark.parametrize("world", [2, 4, 8])
def test_fused_layer_multi_gpu(world):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    _run(world, 29600 + world)


@pytest.mark.parametrize("world", [2, 4])
def test_shadow_and_rebalance_multi_gpu(world):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    _run(world, 29700 + world, worker="mgpu_features_worker.py", token="MGPU_FEATURES_OK", timeout=300)


@pytest.mark.parametrize("world", [2, 4])
def test_expert_parallel_inside_data_parallel_multi_gpu(world):
    """Expert-parallel groups of two ranks inside the job (with 4 ranks: two replicas of every expert, whose gradients
    are reduced over the data-parallel group)."""
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    _run(world, 29710 + world, worker="mgpu_features_worker.py", token="MGPU_EPDP_OK", timeout=300, args=["--ep-inside-dp"])


@pytest.mark.parametrize("world", [2, 4])
def test_sgd_in_the_weight_gradient_epilogue_across_ranks_multi_gpu(world):
    """MoELayer.fuse_sgd on a layer that spans ranks: second projection updated in place, same weights as the ordinary
    path after one step."""
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    _run(world, 29720 + world, worker="mgpu_features_worker.py", token="MGPU_FSGD_OK", timeout=300, args=["--fused-sgd"])
