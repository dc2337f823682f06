"""Autograd-aware entry points of the bandwidth-bound kernels (``elf_b200/csrc/fused_ops.cu``)
with plain-torch implementations of the same math for CPU tensors and other dtypes.

These take the place of the ATen ops the reference's model zoo calls (LayerNorm, GELU,
softmax/cross-entropy, embedding; ``benchmarks/models/simple.py:305-524``) in the
Llama-style models, which need RMSNorm, RoPE and SwiGLU instead.
"""

from __future__ import annotations

from typing import Tuple

import torch
import torch.nn.functional as F

from . import _ext
from .gemm import _ENABLED as _GEMM_ENABLED  # noqa: F401
from . import gemm as _gemm

__all__ = [
    "rms_norm",
    "add_rms_norm",
    "rope_",
    "rope_tables",
    "swiglu",
    "cross_entropy",
    "embedding",
    "kernels_apply",
]


def kernels_apply(t: torch.Tensor) -> bool:
    """The CUDA kernels handle contiguous bf16 CUDA tensors; everything else uses torch."""
    if not (t.is_cuda and t.dtype == torch.bfloat16 and _gemm._ENABLED):
        return False
    _ext.require_on_gpu()
    return True


# ------------------------------------------------------------------------------ RMSNorm
def _rms_ref(x, w, eps):
    xf = x.float()
    rstd = torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
    return (xf * rstd * w.float()).to(x.dtype), rstd.squeeze(-1)


class _RMSNorm(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, eps):
        x = x.contiguous()
        y, rstd, _ = _ext.get().rmsnorm_fwd(x, w, eps, None)
        ctx.save_for_backward(x, w, rstd)
        return y

    @staticmethod
    def backward(ctx, dy):
        x, w, rstd = ctx.saved_tensors
        dw = torch.empty(w.numel(), dtype=torch.float32, device=w.device)
        dx = _ext.get().rmsnorm_bwd(dy.contiguous(), x, w, rstd, dw, False, None, None)
        return dx, dw.to(w.dtype), None


class _AddRMSNorm(torch.autograd.Function):
    """``h = x + residual; y = rmsnorm(h)``; returns ``(y, h)``."""

    @staticmethod
    def forward(ctx, x, residual, w, eps):
        y, rstd, h = _ext.get().rmsnorm_fwd(x.contiguous(), w, eps, residual.contiguous())
        ctx.save_for_backward(h, w, rstd)
        return y, h

    @staticmethod
    def backward(ctx, dy, dh):
        h, w, rstd = ctx.saved_tensors
        dw = torch.empty(w.numel(), dtype=torch.float32, device=w.device)
        dres = None if dh is None else dh.contiguous()
        if dy is None:
            return dh, dh, None, None
        d = _ext.get().rmsnorm_bwd(dy.contiguous(), h, w, rstd, dw, False, dres, None)
        return d, d, dw.to(w.dtype), None


def rms_norm(x: torch.Tensor, w: torch.Tensor, eps: float = 1e-5) -> torch.Tensor:
    if kernels_apply(x) and x.shape[-1] % 8 == 0 and x.shape[-1] <= 8192:
        return _RMSNorm.apply(x, w, eps)
    return _rms_ref(x, w, eps)[0]


def add_rms_norm(x: torch.Tensor, residual: torch.Tensor, w: torch.Tensor, eps: float = 1e-5) -> Tuple[torch.Tensor, torch.Tensor]:
    """Fused residual add + RMSNorm: returns ``(rmsnorm(x + residual), x + residual)``."""
    if kernels_apply(x) and x.shape[-1] % 8 == 0 and x.shape[-1] <= 8192:
        return _AddRMSNorm.apply(x, residual, w, eps)
    h = x + residual
    return _rms_ref(h, w, eps)[0], h


# ------------------------------------------------------------------------------ RoPE
def rope_tables(seq_len: int, head_dim: int, theta: float, device=None) -> Tuple[torch.Tensor, torch.Tensor]:
    """fp32 ``cos, sin`` of shape ``[seq_len, head_dim // 2]`` with ``inv_freq_i = theta^(-2i/d)``."""
    inv = 1.0 / (theta ** (torch.arange(0, head_dim, 2, dtype=torch.float64) / head_dim))
    ang = torch.outer(torch.arange(seq_len, dtype=torch.float64), inv)
    return ang.cos().float().to(device), ang.sin().float().to(device)


def _rope_ref(x2d, cos, sin, n_rot_heads, head_dim, seq_len, sign):
    rows = x2d.shape[0]
    half = head_dim // 2
    pos = torch.arange(rows, device=x2d.device) % seq_len
    c = cos[pos][:, None, :].to(torch.float32)
    s = sin[pos][:, None, :].to(torch.float32) * sign
    rot = x2d[:, : n_rot_heads * head_dim].reshape(rows, n_rot_heads, head_dim).float()
    a, b = rot[..., :half], rot[..., half:]
    out = torch.cat([a * c - b * s, b * c + a * s], dim=-1).reshape(rows, -1).to(x2d.dtype)
    return torch.cat([out, x2d[:, n_rot_heads * head_dim :]], dim=-1)


class _Rope(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x2d, cos, sin, n_rot_heads, head_dim, seq_len):
        ctx.save_for_backward(cos, sin)
        ctx.geom = (n_rot_heads, head_dim, seq_len)
        _ext.get().rope_(x2d, cos, sin, n_rot_heads, head_dim, seq_len, False)
        ctx.mark_dirty(x2d)
        return x2d

    @staticmethod
    def backward(ctx, g):
        cos, sin = ctx.saved_tensors
        n_rot_heads, head_dim, seq_len = ctx.geom
        g = g.clone(memory_format=torch.contiguous_format)  # incoming gradients are not ours to overwrite
        _ext.get().rope_(g, cos, sin, n_rot_heads, head_dim, seq_len, True)
        return g, None, None, None, None, None


def rope_(x2d: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, n_rot_heads: int, head_dim: int, seq_len: int) -> torch.Tensor:
    """Rotate the first ``n_rot_heads`` heads of ``x2d [tokens, heads*head_dim]`` (half-split
    pairing ``(i, i + d/2)``); position = ``row % seq_len``.  In place on the CUDA path."""
    if kernels_apply(x2d) and head_dim % 16 == 0 and x2d.stride(1) == 1:
        return _Rope.apply(x2d, cos, sin, n_rot_heads, head_dim, seq_len)
    return _rope_ref(x2d, cos, sin, n_rot_heads, head_dim, seq_len, 1.0)


# ------------------------------------------------------------------------------ SwiGLU
class _SwiGLU(torch.autograd.Function):
    @staticmethod
    def forward(ctx, gu):
        gu = gu.contiguous()
        ctx.save_for_backward(gu)
        return _ext.get().swiglu_fwd(gu)

    @staticmethod
    def backward(ctx, dout):
        (gu,) = ctx.saved_tensors
        return _ext.get().swiglu_bwd(dout.contiguous(), gu)


def swiglu(gate_up: torch.Tensor) -> torch.Tensor:
    """``silu(gate) * up`` for ``gate_up = [gate | up]`` concatenated on the last dim."""
    if kernels_apply(gate_up) and gate_up.shape[-1] % 16 == 0:
        return _SwiGLU.apply(gate_up)
    g, u = gate_up.chunk(2, dim=-1)
    return F.silu(g) * u


# ------------------------------------------------------------------------------ cross entropy
class _CrossEntropy(torch.autograd.Function):
    """Sum (or mean) of row losses over bf16 logits.  The backward writes
    ``softmax − onehot`` over the logits buffer itself and returns it as the gradient, so
    no second vocabulary-sized tensor is ever allocated."""

    @staticmethod
    def forward(ctx, logits2d, targets, scale, ignore_index):
        loss, lse = _ext.get().ce_fwd(logits2d, targets, ignore_index)
        ctx.save_for_backward(logits2d, targets, lse)
        ctx.scale, ctx.ignore_index = scale, ignore_index
        return loss.sum() * scale

    @staticmethod
    def backward(ctx, g):
        logits2d, targets, lse = ctx.saved_tensors
        gs = g.detach().to(torch.float32).reshape(1).contiguous()
        _ext.get().ce_bwd(logits2d, logits2d, targets, lse, gs, ctx.scale, ctx.ignore_index)
        return logits2d, None, None, None


def cross_entropy(logits: torch.Tensor, target: torch.Tensor, reduction: str = "mean", ignore_index: int = -100) -> torch.Tensor:
    """Token cross entropy in fp32 math.  ``logits [..., vocab]``, ``target [...]``.

    On the CUDA path the logits buffer is consumed: after ``backward`` it holds the
    gradient.  Callers that still need the logits must clone them first."""
    vocab = logits.shape[-1]
    flat_t = target.reshape(-1)
    if kernels_apply(logits) and reduction in ("sum", "mean") and logits.is_contiguous() and vocab % 8 == 0:
        n = flat_t.numel()
        if reduction == "mean":
            valid = (flat_t != ignore_index).sum().clamp_min(1).item() if ignore_index >= 0 else n
            scale = 1.0 / max(valid, 1)
        else:
            scale = 1.0
        return _CrossEntropy.apply(logits.view(-1, vocab), flat_t.contiguous(), scale, ignore_index)
    return F.cross_entropy(logits.float().reshape(-1, vocab), flat_t, reduction=reduction, ignore_index=ignore_index)


# ------------------------------------------------------------------------------ embedding
class _Embedding(torch.autograd.Function):
    """Gather forward; the backward sorts the token ids (4 k integers) and sums the output
    gradient rows of each token in order - deterministic, no atomics.  With ``into_grad`` the sums
    are added straight into ``table.grad`` (or ``table.main_grad``), which is how the pipeline
    runs it: no dense ``[vocab, dim]`` temporary per micro-batch."""

    @staticmethod
    def forward(ctx, table, ids, into_grad):
        ctx.save_for_backward(ids)
        ctx.table = table if into_grad else None
        ctx.shape = table.shape
        from . import gemm as _gemm

        # an id outside the table reads nothing (zero row) and leaves a record that the optimizer
        # step and the next pipeline step raise on
        return _ext.get().embedding_fwd(table, ids.contiguous(), _gemm.status(table.device))

    @staticmethod
    def backward(ctx, dout):
        (ids,) = ctx.saved_tensors
        sorted_ids, perm = torch.sort(ids.reshape(-1), stable=True)
        table = ctx.table
        if table is not None:
            target = getattr(table, "main_grad", None)
            if target is None:
                if table.grad is None:
                    table.grad = torch.zeros_like(table)
                target = table.grad
            if target.is_contiguous() and target.dtype in (torch.bfloat16, torch.float32):
                _ext.get().embedding_bwd_sorted(dout.contiguous(), sorted_ids, perm, target)
                return None, None, None
        dtable = torch.zeros(ctx.shape, dtype=dout.dtype, device=dout.device)
        _ext.get().embedding_bwd_sorted(dout.contiguous(), sorted_ids, perm, dtable)
        return dtable, None, None


def embedding(table: torch.Tensor, ids: torch.Tensor, into_grad: bool = False) -> torch.Tensor:
    """``table[ids]``.  ``into_grad=True`` (for parameters): the backward accumulates into
    ``table.grad`` in place instead of handing autograd a dense gradient."""
    if kernels_apply(table) and table.shape[1] % 8 == 0 and table.is_contiguous():
        return _Embedding.apply(table, ids, bool(into_grad) and table.requires_grad and table.is_leaf)
    return F.embedding(ids, table)
