"""tcgen05 GEMM family for linear layers (kernels in ``elf_b200/csrc/gemm_sm100.cu``).

=====================  ==============================  ===================================
pass                   product                         operand layouts fed to the kernel
=====================  ==============================  ===================================
forward                ``Y[M,N]  = X[M,K] · W[N,K]ᵀ``  A = X K-major,   B = W K-major
input grad  (B pass)   ``dX[M,K] = dY[M,N] · W[N,K]``  A = dY K-major,  B = W MN-major
weight grad (W pass)   ``dW[N,K] (+)= dY[M,N]ᵀ · X``   A = dY MN-major, B = X MN-major
=====================  ==============================  ===================================

No operand is ever transposed in memory: "MN-major" tiles are fetched by TMA as 64-wide
boxes and described to the tensor core as such.  These replace the cuBLAS calls behind
``F.linear`` / ``torch.mm`` in the reference (``elf/zb_utils.py:20,35-37,236-238``) and the
separate ``grad.add_`` pass (``:241-252``): accumulation happens in the epilogue.
"""

from __future__ import annotations

import os
from typing import Dict, Optional

import torch

from . import _ext

__all__ = [
    "usable",
    "grad_buffer_ok",
    "linear_forward",
    "linear_input_grad",
    "linear_weight_grad",
    "matmul_nt",
    "status",
    "check_status",
    "snapshot_status_async",
    "raise_if_failed",
    "set_enabled",
    "set_variant",
]

_ENABLED = os.environ.get("ELF_B200_DISABLE_KERNELS", "0") != "1"
# 0 = one CTA per 128x256 tile, 1 = CTA pairs (cta_group::2) on 256x256 tiles
_VARIANT = int(os.environ.get("ELF_B200_GEMM_VARIANT", "1"))
# split the tiles of the last, partly filled wave (pair kernel: along K with partial sums added in L2; 1-CTA kernel: into column strips)
_SPLIT_TAIL = os.environ.get("ELF_B200_GEMM_SPLIT_TAIL", "1") != "0"
_STATUS: Dict[int, torch.Tensor] = {}
_DTYPES = (torch.bfloat16, torch.float16)


def set_enabled(flag: bool) -> None:
    """Switch the kernels off (torch ops are used instead) — for A/B numerics tests."""
    global _ENABLED
    _ENABLED = bool(flag)


def set_variant(variant: int, split_tail: bool = True) -> None:
    """Select the kernel variant (0 single CTA, 1 CTA pair) and the tail-wave splitting."""
    global _VARIANT, _SPLIT_TAIL
    _VARIANT, _SPLIT_TAIL = int(variant), bool(split_tail)


def status(device=None) -> torch.Tensor:
    """Per-device int32[4] error record the kernels write on a bounded-wait timeout."""
    if isinstance(device, int):
        idx = device
    else:
        idx = torch.cuda.current_device() if device is None else torch.device(device).index or 0
    if idx not in _STATUS:
        _STATUS[idx] = torch.zeros(4, dtype=torch.int32, device=f"cuda:{idx}")
    return _STATUS[idx]


def check_status(device=None) -> None:
    """Synchronising check: raise if any kernel on ``device`` recorded an error."""
    rec = status(device).tolist()
    if rec[0] != 0:
        status(device).zero_()
        what = _WHAT.get(rec[0], "unknown")
        raise RuntimeError(f"elf_b200 kernel error {rec[0]} ({what}); detail={rec[1:]}")


_SNAPSHOT: Dict[int, tuple] = {}  # device index -> (pinned int32[4], event of the last copy into it)
_WHAT = {1: "an mbarrier wait timed out", 2: "a wait on a peer GPU timed out", 3: "bad shape", 4: "an index outside its table (detail: 1 forward / 2 backward, row, index)"}


def snapshot_status_async(device=None) -> None:
    """Queue a copy of the device's error record into pinned host memory on the current
    stream (16 bytes, no synchronisation).  ``raise_if_failed`` later looks at the copy."""
    if not torch.cuda.is_available():
        return
    idx = torch.cuda.current_device() if device is None else (torch.device(device).index or 0)
    if idx not in _STATUS:
        return  # no kernel of this package has been given a status word on this device yet
    entry = _SNAPSHOT.get(idx)
    if entry is None:
        entry = _SNAPSHOT[idx] = (torch.zeros(4, dtype=torch.int32).pin_memory(), torch.cuda.Event())
    host, event = entry
    with torch.cuda.device(idx):
        host.copy_(_STATUS[idx], non_blocking=True)
        event.record()


def raise_if_failed(device=None) -> None:
    """Non-blocking check of the last completed ``snapshot_status_async``: raises when a
    kernel of an earlier step recorded an error (a bounded wait that ran out).  Called at the
    start of ``Pipeline.step`` and ``FusedAdamW.step``; after an error the optimizer kernel
    has skipped its update, so parameters are still those of the last good step."""
    if not _SNAPSHOT:
        return
    idx = torch.cuda.current_device() if device is None else (torch.device(device).index or 0)
    entry = _SNAPSHOT.get(idx)
    if entry is None:
        return
    host, event = entry
    if not event.query():
        return  # the copy has not landed yet; the next call will see it
    rec = host.tolist()
    if rec[0] != 0:
        host.zero_()
        status(idx).zero_()
        raise RuntimeError(f"elf_b200 kernel error {rec[0]} ({_WHAT.get(rec[0], 'unknown')}) in an earlier step; detail={rec[1:]}. "
                           "The optimizer skipped the update of that step; gradients of that step are not valid.")


def usable(x: torch.Tensor, w: torch.Tensor) -> bool:
    """Whether the tcgen05 path applies to this (activation, weight) pair."""
    if not (x.is_cuda and w.is_cuda and _ENABLED):
        return False
    if x.dtype not in _DTYPES or w.dtype != x.dtype or w.dim() != 2:
        return False
    _ext.require_on_gpu()
    n, k = w.shape
    return n % 8 == 0 and k % 8 == 0 and x.shape[-1] in (n, k) and x.numel() > 0


def grad_buffer_ok(weight: torch.Tensor) -> bool:
    g = weight.grad
    return g is None or (g.is_contiguous() and g.dtype in (weight.dtype, torch.float32) and g.shape == weight.shape)


def _rows(t: torch.Tensor) -> torch.Tensor:
    t2 = t.reshape(-1, t.shape[-1])
    if t2.stride(-1) != 1 or (t2.stride(0) * t2.element_size()) % 16 or t2.data_ptr() % 16:
        t2 = t2.contiguous()
    return t2


def linear_forward(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    x2 = _rows(x)
    # allocated in its final shape: the result must not be a view made inside an autograd
    # Function, or later in-place ops on it (RoPE) would be rejected
    y = torch.empty((*x.shape[:-1], w.shape[0]), dtype=x.dtype, device=x.device)
    b = None if bias is None else bias.to(x.dtype).contiguous()
    _ext.get().gemm(x2, _rows(w), y.view(-1, w.shape[0]), b, False, False, False, 1.0, status(x.device), _VARIANT, _SPLIT_TAIL)
    return y


def linear_input_grad(dy: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    dy2 = _rows(dy)
    dx = torch.empty((*dy.shape[:-1], w.shape[1]), dtype=dy.dtype, device=dy.device)
    _ext.get().gemm(dy2, _rows(w), dx.view(-1, w.shape[1]), None, False, True, False, 1.0, status(dy.device), _VARIANT, _SPLIT_TAIL)
    return dx


def linear_weight_grad(dy: torch.Tensor, x: torch.Tensor, out: Optional[torch.Tensor] = None, alpha: float = 1.0, out_dtype=None, push: Optional[dict] = None) -> torch.Tensor:
    """``out (+)= alpha · dyᵀ·x``; accumulates when ``out`` is given, else allocates
    (``out_dtype`` defaults to the operand dtype).  ``push`` (peer addresses, flag addresses,
    flag value, counter; see ``elf_b200.parallel.dp_sync``) makes the epilogue also store the
    result into peer GPUs' memory and flag it there."""
    dy2, x2 = _rows(dy), _rows(x)
    accumulate = out is not None
    if out is None:
        out = torch.empty((dy2.shape[1], x2.shape[1]), dtype=out_dtype or dy.dtype, device=dy.device)
    if push:
        _ext.get().gemm(dy2, x2, out, None, True, True, accumulate, float(alpha), status(dy.device), _VARIANT, _SPLIT_TAIL,
                        push["push_out"], push["push_flags"], push["push_flag_value"], push["push_counter"])
    else:
        _ext.get().gemm(dy2, x2, out, None, True, True, accumulate, float(alpha), status(dy.device), _VARIANT, _SPLIT_TAIL)
    return out


def matmul_nt(a: torch.Tensor, b: torch.Tensor, out_dtype=None) -> torch.Tensor:
    """``a[M,K] · b[N,K]ᵀ`` for plain 2-D use."""
    a2, b2 = _rows(a), _rows(b)
    d = torch.empty((a2.shape[0], b2.shape[0]), dtype=out_dtype or a.dtype, device=a.device)
    _ext.get().gemm(a2, b2, d, None, False, False, False, 1.0, status(a.device), _VARIANT, _SPLIT_TAIL)
    return d
