"""Multi-GPU correctness (2 GPUs by default), each case a torchrun child job."""

import os
import subprocess
import sys

import pytest
import torch

pytestmark = [pytest.mark.gpu, pytest.mark.multigpu]

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def launch(case: str, nproc: int, timeout: int = 240, **extra_env):
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", **extra_env)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}", "--master-addr", "127.0.0.1",
           "--master-port", str(29600 + (os.getpid() % 300)), os.path.join(ROOT, "tests", "multigpu_worker.py"), case]
    out = subprocess.run(cmd, cwd=ROOT, env=env, capture_output=True, text=True, timeout=timeout)
    assert out.returncode == 0, out.stdout[-3000:] + "\n" + out.stderr[-6000:]
    assert out.stdout.count(f"case {case} ok") == nproc, out.stdout[-2000:]


def test_peer_memory_gradient_exchange_matches_allreduce():
    launch("dp_symm", 2)


def test_pipeline_zbv_two_gpus():
    launch("pp", 2)


def test_pipeline_stages_cut_inside_layers_two_gpus():
    launch("pp_split", 2)


def test_pipeline_copy_engine_transport_two_gpus():
    launch("pp_copy", 2)


def test_own_symmetric_memory_runtime_under_gradient_exchange_and_copy_transport():
    """The same two cases with the buffers allocated, exported and mapped by this package's
    runtime on CUDA virtual memory (``ELF_B200_SYMM=vmm``) instead of torch's symmetric memory."""
    launch("dp_symm", 2, ELF_B200_SYMM="vmm")
    launch("pp_copy", 2, ELF_B200_SYMM="vmm")


@pytest.mark.skipif(torch.cuda.device_count() < 4, reason="needs 4 GPUs")
def test_pipeline_copy_engine_transport_four_gpus():
    """Middle ranks have two neighbours: the arenas of all ranks are mapped in one rendezvous."""
    launch("pp_copy", 4)


@pytest.mark.skipif(torch.cuda.device_count() < 4, reason="needs 4 GPUs")
def test_pipeline_with_replicas_four_gpus():
    launch("pp_dp", 4)
