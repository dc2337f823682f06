"""Causal grouped-query attention.

``attention(q, k, v)`` takes ``q [B, S, Hq, D]`` and ``k, v [B, S, Hkv, D]`` (any strides with a
contiguous head dim — e.g. slices of one fused QKV projection) and returns ``[B, S, Hq, D]``.
Back ends: on CUDA with bf16, head dimension 128 and a sequence length that is a multiple of 128
the packed entry point runs this package's tcgen05 forward kernel (``attention_native.py``); its
backward is the library's fused kernel fed with our output and log-sum-exp unless
``ELF_B200_ATTENTION_BACKWARD=native`` selects the own backward kernels.  Everything else, and
``ELF_B200_ATTENTION=library``, goes through ``torch.nn.functional.scaled_dot_product_attention``
(a library call, also what the reference's model zoo uses,
``benchmarks/models/simple.py:14-25,381-386``).
"""

from __future__ import annotations

import torch
import torch.nn.functional as F

from . import _ext
from . import gemm as _gemm

__all__ = ["attention", "attention_packed", "native_available"]


def native_available() -> bool:
    return _ext.available() and hasattr(_ext.get(), "attention_fwd")


def _sdpa(q, k, v, causal: bool):
    qh, kh, vh = q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2)
    out = F.scaled_dot_product_attention(qh, kh, vh, is_causal=causal, enable_gqa=qh.shape[1] != kh.shape[1])
    return out.transpose(1, 2)


class _PackedSDPA(torch.autograd.Function):
    """Attention over a fused ``qkv [B, S, Hq + 2 Hkv, D]`` buffer through the library SDPA.

    Slicing q/k/v out of the buffer under autograd would make every backward allocate three
    zero-filled full-size tensors and add them up; here the three gradients are written
    once into one ``dqkv`` buffer."""

    @staticmethod
    def forward(ctx, qkv, hq, hkv, causal):
        base = qkv.detach()
        with torch.enable_grad():
            q = base[:, :, :hq].requires_grad_()
            k = base[:, :, hq : hq + hkv].requires_grad_()
            v = base[:, :, hq + hkv :].requires_grad_()
            out = _sdpa(q, k, v, causal)
        ctx.graph = (q, k, v, out)
        ctx.hq, ctx.hkv = hq, hkv
        ctx.save_for_backward(qkv)  # lets checkpointing / offload see the dependency
        return out.detach()

    @staticmethod
    def backward(ctx, g):
        q, k, v, out = ctx.graph
        ctx.graph = None
        dq, dk, dv = torch.autograd.grad(out, (q, k, v), g)
        (qkv,) = ctx.saved_tensors
        dqkv = torch.empty_like(qkv)
        hq, hkv = ctx.hq, ctx.hkv
        dqkv[:, :, :hq].copy_(dq)
        dqkv[:, :, hq : hq + hkv].copy_(dk)
        dqkv[:, :, hq + hkv :].copy_(dv)
        return dqkv, None, None, None


def attention_packed(qkv: torch.Tensor, n_heads: int, n_kv_heads: int, causal: bool = True) -> torch.Tensor:
    """``qkv [B, S, Hq + 2 Hkv, D]`` → ``[B, S, Hq, D]``."""
    if qkv.is_cuda and _gemm._ENABLED:
        if native_available():
            from .attention_native import native_attention_packed, native_applicable_packed

            if native_applicable_packed(qkv, n_heads, n_kv_heads, causal):
                return native_attention_packed(qkv, n_heads, n_kv_heads)
        return _PackedSDPA.apply(qkv, n_heads, n_kv_heads, causal)
    q, k, v = qkv[:, :, :n_heads], qkv[:, :, n_heads : n_heads + n_kv_heads], qkv[:, :, n_heads + n_kv_heads :]
    return _sdpa(q, k, v, causal)


def attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, causal: bool = True) -> torch.Tensor:
    if q.is_cuda and _gemm._ENABLED and native_available():
        from .attention_native import native_attention, native_applicable

        if native_applicable(q, k, v, causal):
            return native_attention(q, k, v)
    return _sdpa(q, k, v, causal)
