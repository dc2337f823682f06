"""Causal grouped-query attention.

``attention(q, k, v)`` takes ``q [B, S, Hq, D]`` and ``k, v [B, S, Hkv, D]`` (any strides with a
contiguous head dim — e.g. slices of one fused QKV projection) and returns ``[B, S, Hq, D]``.
Back ends, in order: this package's sm_100a kernel when built and applicable, else
``torch.nn.functional.scaled_dot_product_attention`` (a library call, also what the
reference's model zoo uses, ``benchmarks/models/simple.py:14-25,381-386``).
"""

from __future__ import annotations

import torch
import torch.nn.functional as F

from . import _ext
from . import gemm as _gemm

__all__ = ["attention", "native_available"]


def native_available() -> bool:
    return _ext.available() and hasattr(_ext.get(), "attention_fwd")


def _sdpa(q, k, v, causal: bool):
    qh, kh, vh = q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2)
    out = F.scaled_dot_product_attention(qh, kh, vh, is_causal=causal, enable_gqa=qh.shape[1] != kh.shape[1])
    return out.transpose(1, 2)


def attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, causal: bool = True) -> torch.Tensor:
    if q.is_cuda and _gemm._ENABLED and native_available():
        from .attention_native import native_attention, native_applicable

        if native_applicable(q, k, v, causal):
            return native_attention(q, k, v)
    return _sdpa(q, k, v, causal)
