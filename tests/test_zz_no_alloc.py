"""The allocation-free RMSNorm backward (``elf_b200/csrc/rmsnorm_bwd_noalloc.h``).

That entry point is meant for callers that must not allocate device memory while they run -
a stage executing under a memory plan fixed in advance, or a C/C++ host without PyTorch's
caching allocator - so it keeps its column-sum scratch in a fixed array inside the library.
It is called here the way such a caller would: through the exported C symbol of the
stand-alone shared library, with raw device pointers.  Its results must agree with the
regular entry point (which takes its scratch from the allocator) on two calls in a row; the
second call uses other data and a smaller shape, so stale scratch contents would show.

This file sorts last on purpose: a run that stops at the first failure has then already run
every other test."""

import ctypes
import os

import pytest
import torch

pytestmark = pytest.mark.gpu

LIB = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "elf_b200", "csrc", "_build", "libelfb_noalloc.so")


def _load():
    assert os.path.exists(LIB), f"{LIB} is missing: run `python -m elf_b200.csrc.build`"
    lib = ctypes.CDLL(LIB)
    lib.elfb_rmsnorm_backward_noalloc.restype = ctypes.c_int
    lib.elfb_rmsnorm_backward_noalloc.argtypes = [ctypes.c_void_p] * 6 + [ctypes.c_int, ctypes.c_int, ctypes.c_void_p]
    lib.elfb_noalloc_last_error.restype = ctypes.c_char_p
    return lib


def _case(rows, dim, seed, dev):
    from elf_b200.ops import _ext

    g = torch.Generator(device=dev).manual_seed(seed)
    x = torch.randn(rows, dim, device=dev, generator=g).to(torch.bfloat16)
    dy = torch.randn(rows, dim, device=dev, generator=g).to(torch.bfloat16)
    w = (1 + 0.1 * torch.randn(dim, device=dev, generator=g)).to(torch.bfloat16)
    _, rstd, _ = _ext.get().rmsnorm_fwd(x, w, 1e-5, None)
    return x, dy, w, rstd


def test_no_alloc_entry_point_matches_regular_path_twice():
    from elf_b200.ops import _ext

    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    lib = _load()
    stream = torch.cuda.current_stream(dev)
    # set-up call: the first use on a device resolves the scratch array's address, and the driver
    # gives the library's static array (2 MiB) its memory when the module is first used; from then
    # on no call may change the amount of free device memory
    x0, dy0, w0, rstd0 = _case(8, 64, 1, dev)
    dx0, dw0 = torch.empty_like(x0), torch.empty(64, device=dev)
    assert lib.elfb_rmsnorm_backward_noalloc(dy0.data_ptr(), x0.data_ptr(), w0.data_ptr(), rstd0.data_ptr(), dx0.data_ptr(), dw0.data_ptr(), 8, 64, stream.cuda_stream) == 0
    torch.cuda.synchronize(dev)
    # the second case is the documented maximum width (whole scratch array, wide-row kernel variant);
    # the third, narrower one would show scratch contents left over from it
    for call, (rows, dim, seed) in enumerate([(300, 4096, 11), (70, 8192, 13), (77, 1024, 12)]):
        x, dy, w, rstd = _case(rows, dim, seed, dev)
        # regular entry point: scratch comes from torch's allocator
        dw_ref = torch.empty(dim, device=dev, dtype=torch.float32)
        dx_ref = _ext.get().rmsnorm_bwd(dy, x, w, rstd, dw_ref, False, None, None)
        # allocation-free entry point: outputs are ours, scratch is inside the library
        dx = torch.empty_like(x)
        dw = torch.full((dim,), float("nan"), device=dev, dtype=torch.float32)
        torch.cuda.synchronize(dev)
        before = torch.cuda.memory_allocated(dev)
        free_before, _ = torch.cuda.mem_get_info(dev)  # the driver's view: sees a cudaMalloc that torch's counters cannot
        rc = lib.elfb_rmsnorm_backward_noalloc(dy.data_ptr(), x.data_ptr(), w.data_ptr(), rstd.data_ptr(), dx.data_ptr(), dw.data_ptr(), rows, dim, stream.cuda_stream)
        assert rc == 0, lib.elfb_noalloc_last_error().decode()
        torch.cuda.synchronize(dev)
        assert torch.cuda.memory_allocated(dev) == before
        assert torch.cuda.mem_get_info(dev)[0] >= free_before, "device memory was allocated behind the entry point"
        torch.testing.assert_close(dx.float(), dx_ref.float(), atol=1e-2, rtol=1e-2, msg=lambda m: f"call {call}: dx {m}")
        torch.testing.assert_close(dw, dw_ref, atol=1e-2, rtol=1e-2, msg=lambda m: f"call {call}: dw {m}")
        # and against plain fp32 math, like the other kernel tests
        xf, wf = x.float().requires_grad_(), w.float().requires_grad_()
        torch.nn.functional.rms_norm(xf, (dim,), wf, 1e-5).backward(dy.float())
        assert ((dx.float() - xf.grad).norm() / xf.grad.norm()).item() < 1e-2
        assert ((dw - wf.grad).norm() / wf.grad.norm()).item() < 1e-2


def test_no_alloc_entry_point_rejects_what_does_not_fit():
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    lib = _load()
    x, dy, w, rstd = _case(8, 64, 1, dev)
    dx, dw = torch.empty_like(x), torch.empty(64, device=dev)
    args = (dy.data_ptr(), x.data_ptr(), w.data_ptr(), rstd.data_ptr(), dx.data_ptr(), dw.data_ptr())
    assert lib.elfb_rmsnorm_backward_noalloc(*args, 8, 8192 + 8, None) == -1
    assert b"maximum 8192" in lib.elfb_noalloc_last_error()
    assert lib.elfb_rmsnorm_backward_noalloc(*args, 8, 60, None) == -1
    assert lib.elfb_rmsnorm_backward_noalloc(None, *args[1:], 8, 64, None) == -2
    assert lib.elfb_rmsnorm_backward_noalloc(args[0] + 2, *args[1:], 8, 64, None) == -2  # pointer off its 16-byte boundary
    assert b"aligned" in lib.elfb_noalloc_last_error()
    assert lib.elfb_rmsnorm_backward_noalloc(*args, 0, 64, None) == 0  # no rows: nothing to do, nothing launched
    assert lib.elfb_rmsnorm_backward_noalloc(*args, 8, 64, None) == 0
    torch.cuda.synchronize(dev)
