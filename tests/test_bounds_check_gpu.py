"""The bounds-checking variant of the extension (``-DELF_BOUNDS_CHECK``, loaded with
``ELF_B200_BOUNDS_CHECK=1``): correct kernels leave the status word alone, a copy with
forbidden coordinates is recorded and skipped.  Runs in a child process because a process can
hold only one variant of the extension."""

import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

CHILD = r"""
import torch
from elf_b200.ops import _ext, gemm
from elf_b200.ops import attention_native as an

ext = _ext.get()
assert ext.bounds_check_build(), "the regular build was loaded"
dev = torch.device("cuda", 0)
torch.manual_seed(0)

def rel(a, b):
    return ((a.float() - b.float()).norm() / b.float().norm().clamp_min(1e-12)).item()

# GEMM family on a ragged shape: forward, input gradient, weight gradient added to what is there
x = torch.randn(520, 328, device=dev).bfloat16()
w = torch.randn(264, 328, device=dev).bfloat16()
dy = torch.randn(520, 264, device=dev).bfloat16()
assert rel(gemm.linear_forward(x, w), x.float() @ w.float().t()) < 1e-2
assert rel(gemm.linear_input_grad(dy, w), dy.float() @ w.float()) < 1e-2
grad = torch.ones_like(w)
gemm.linear_weight_grad(dy, x, out=grad)
assert rel(grad, dy.float().t() @ x.float() + 1.0) < 1e-2

# attention forward (TMA loads of Q, K, V tiles)
b, s, hq, hkv, d = 1, 256, 4, 2, 128
qkv = torch.randn(b, s, hq + 2 * hkv, d, device=dev).bfloat16()
assert an.native_applicable_packed(qkv, hq, hkv, True)
out, lse = an.forward_packed(qkv, hq, hkv)
q, k, v = qkv[:, :, :hq], qkv[:, :, hq:hq + hkv], qkv[:, :, hq + hkv:]
ref = torch.nn.functional.scaled_dot_product_attention(q.transpose(1, 2).float(), k.transpose(1, 2).float().repeat_interleave(hq // hkv, 1),
                                                       v.transpose(1, 2).float().repeat_interleave(hq // hkv, 1), is_causal=True).transpose(1, 2)
assert rel(out.view(b, s, hq, d), ref) < 2e-2
torch.cuda.synchronize()
assert gemm.status(dev).tolist()[0] == 0, gemm.status(dev).tolist()

# two copies with forbidden coordinates: recorded (first one: where 4 = store, x 3, y 0), not issued
ext.bounds_check_selftest(gemm.status(dev))
torch.cuda.synchronize()
assert gemm.status(dev).tolist() == [5, 4, 3, 0], gemm.status(dev).tolist()
gemm.status(dev).zero_()
# the device is healthy afterwards
assert rel(gemm.linear_forward(x, w), x.float() @ w.float().t()) < 1e-2
torch.cuda.synchronize()
assert gemm.status(dev).tolist()[0] == 0
print("bounds-check build ok")
"""


def test_bounds_check_build_passes_clean_kernels_and_records_a_forbidden_copy():
    so = os.path.join(ROOT, "elf_b200", "csrc", "_build_check", "elf_b200_C_check.so")
    assert os.path.exists(so), "build the variant with `python -m elf_b200.csrc.build --bounds-check`"
    env = dict(os.environ, ELF_B200_BOUNDS_CHECK="1", PYTHONPATH=ROOT + os.pathsep + os.environ.get("PYTHONPATH", ""))
    out = subprocess.run([sys.executable, "-c", CHILD], cwd=ROOT, env=env, capture_output=True, text=True, timeout=300)
    assert out.returncode == 0, out.stdout[-2000:] + out.stderr[-4000:]
    assert "bounds-check build ok" in out.stdout
