"""The scripts under ``examples/`` run as written (CPU ranks over gloo)."""

import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _torchrun(script, nproc, port, *args):
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}", "--master-addr", "127.0.0.1", "--master-port", str(port),
           os.path.join(ROOT, "examples", script), *args]
    out = subprocess.run(cmd, cwd=ROOT, capture_output=True, text=True, timeout=300, env=dict(os.environ, CUDA_VISIBLE_DEVICES=""))
    assert out.returncode == 0, out.stdout[-1500:] + out.stderr[-3000:]
    return out.stdout


@pytest.mark.parametrize("script,nproc", [("basic.py", 2), ("basic_no_partition.py", 2)])
def test_basic_examples(script, nproc):
    out = _torchrun(script, nproc, 29791 if script == "basic.py" else 29792)
    assert "loss" in out


def test_profile_guided_zbv_example():
    out = _torchrun("llama_zbv_profile_guided.py", 2, 29793, "--name", "llama-tiny", "--nmb", "4", "--steps", "3")
    assert out.count("loss") == 3
