"""FLOP formulas for ops ``torch.utils.flop_counter`` does not know
(reference ``elf/utils.py:521-571``), plus closed forms for the transformer ops
this package implements as kernels, used for roofline reporting."""

from __future__ import annotations

import math

import torch
from torch.utils.flop_counter import register_flop_formula

__all__ = ["prod", "linear_flops", "attention_flops", "transformer_step_flops"]

aten = torch.ops.aten


def prod(xs):
    if isinstance(xs, (int, float)):
        return xs
    acc = 1
    for x in xs:
        acc *= x
    return acc


def _register(ops, fn):
    try:
        register_flop_formula(ops)(fn)
    except Exception:  # already registered by another import of the same formulas
        pass
    return fn


def _ewise_binary(a_shape, b_shape=None, *args, out_shape=None, **kwargs) -> int:
    return prod(a_shape)


def _ewise_unary(a_shape, *args, out_shape=None, **kwargs) -> int:
    return prod(a_shape)


def _gelu(x_shape, *args, **kwargs) -> int:
    # x/sqrt2, erf (~30), 1+, x*, 0.5* → about 34 flops per element
    return 34 * prod(x_shape)


def _fft_c2c(x_shape, dim, *args, **kwargs) -> int:
    dims = dim if isinstance(dim, (list, tuple)) else [dim]
    per_line = sum(5 * x_shape[d] * math.log2(x_shape[d]) for d in dims if x_shape[d] > 1)
    lines = prod(x_shape) // prod(x_shape[d] for d in dims)
    return int(per_line * lines)


def _fft_r2c(x_shape, dim, *args, **kwargs) -> int:
    return _fft_c2c(x_shape, dim) // 2


_register([aten.add, aten.mul, aten.sub, aten.div], _ewise_binary)
_register([aten.abs], _ewise_unary)
_register(aten.gelu, _gelu)
_register([aten.gelu_backward], _gelu)
_register([aten._fft_c2c], _fft_c2c)
_register([aten._fft_r2c], _fft_r2c)


def linear_flops(m: int, n: int, k: int) -> int:
    return 2 * m * n * k


def attention_flops(b: int, hq: int, s: int, d: int, causal: bool = True, backward: bool = False) -> int:
    """QKᵀ and PV (forward, 2 GEMMs) or the 5 GEMMs of the backward."""
    gemms = 5 if backward else 2
    f = gemms * 2 * b * hq * s * s * d
    return f // 2 if causal else f


def transformer_step_flops(n_layers, d, n_heads, n_kv_heads, ffn, vocab, seq, tokens, gated=True) -> int:
    """Model FLOPs of one forward+backward over ``tokens`` tokens (3× forward)."""
    hd = d // n_heads
    per_tok = 2 * d * (n_heads + 2 * n_kv_heads) * hd + 2 * d * d + 2 * d * ffn * (3 if gated else 2)
    fwd = tokens * (n_layers * per_tok + 2 * d * vocab)
    fwd += n_layers * attention_flops(tokens // seq, n_heads, seq, hd)
    return 3 * fwd
