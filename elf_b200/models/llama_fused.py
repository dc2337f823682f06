"""Decoder layers (and their halves) as single autograd nodes with hand-written backward passes.

``LlamaDecoderLayer`` written as a chain of small autograd functions (norm, linear, RoPE,
attention, linear, add+norm, linear, SwiGLU, linear, add) makes autograd do work that a
hand-written backward does not need: it clones the gradient before the in-place RoPE
backward, adds the two gradients of every residual branch with a kernel of its own, converts
and accumulates the norm gains' gradients in three more, and runs a dozen Python-level nodes
per layer and direction.  Here a whole layer, or either half of it, is ONE
``torch.autograd.Function``:

``attention_half(x)``  ``x + wo(attention(rope(wqkv(rmsnorm(x)))))``
``mlp_half(x)``        ``x + w_down(swiglu(w_gate_up(rmsnorm(x))))``
``decoder_layer(x)``   both, with the first residual add fused into the second norm

The forward runs the kernels back to back; the backward runs the input-gradient chain by
hand: residual gradients enter the RMSNorm backward kernel as its ``dres`` operand (one pass,
no separate add), RoPE's backward rotates the attention gradient in place (it is ours), and
the norm gains' gradients are accumulated by the kernel straight into the gradient buffer.
The four projections stay ``LinearDW`` layers as far as the runtime is concerned: the
functions file their inputs and output gradients in the layers' staging slots, so the W pass,
its in-epilogue accumulation, the peer push of the data-parallel exchange, rematerialisation
(the functions' saved tensors go through ``save_for_backward``) and the partial backward
replay work as with separate nodes.

Used on CUDA with bf16 tensors; every other case takes the composed path in
``elf_b200.models.llama``.
"""

from __future__ import annotations

import math

import torch

from ..ops import _ext
from ..ops import attention as _attn
from ..ops import fused as _f
from ..ops import gemm as _gemm
from ..zb_utils import LayerDW, in_partial_replay

__all__ = ["fused_apply", "attention_half", "mlp_half", "decoder_layer"]


def fused_apply(x: torch.Tensor, *linears) -> bool:
    """Whether the single-node path applies: bf16 CUDA activations ``[batch, seq, d]``, kernels
    enabled, every projection a bias-free split-backward layer on the tcgen05 path."""
    from ..zb_utils import LinearDW

    if not (_f.kernels_apply(x) and x.dim() == 3 and x.shape[-1] % 8 == 0 and x.shape[-1] <= 8192):
        return False
    if not hasattr(_ext.get(), "residual_add"):
        return False
    for lin in linears:
        if not isinstance(lin, LinearDW) or lin.bias is not None or lin.weight.dtype != x.dtype or not lin.weight.is_cuda:
            return False
        n, k = lin.weight.shape
        if n % 8 or k % 8:
            return False
    return True


def _norm_grad_target(w: torch.Tensor) -> torch.Tensor:
    """Buffer the RMSNorm backward kernel accumulates the gain's gradient into (a throw-away one
    while a partial backward replay refills the W-pass stashes: the gradient is in already)."""
    if in_partial_replay():
        return torch.zeros_like(w)
    target = getattr(w, "main_grad", None)
    if target is None:
        if w.grad is None:
            w.grad = torch.zeros_like(w)
        target = w.grad
    return target


def _stash_input(linear, t: torch.Tensor) -> None:
    stash = t.detach()
    stash.is_model_input = False  # produced inside the node: a checkpointed re-run regenerates it
    linear.last_input = stash


# ---------------------------------------------------------------------------------------
# attention: library or native kernels behind one functional interface
# ---------------------------------------------------------------------------------------

_NATIVE, _LIBRARY = 0, 1


def _attention_forward(qkv: torch.Tensor, hq: int, hkv: int):
    """``qkv [B, S, hq + 2 hkv, D]`` -> ``(out [B, S, hq, D], mode, tensors to save)``."""
    if _attn.native_available():
        from ..ops import attention_native as _n

        if _n.native_applicable_packed(qkv, hq, hkv, True):
            out, lse = _n.forward_packed(qkv, hq, hkv)
            return out, _NATIVE, (lse,)
    q = qkv[:, :, :hq].transpose(1, 2)
    k = qkv[:, :, hq : hq + hkv].transpose(1, 2)
    v = qkv[:, :, hq + hkv :].transpose(1, 2)
    res = torch.ops.aten._scaled_dot_product_cudnn_attention(q, k, v, None, True, 0.0, True, False)
    return res[0].transpose(1, 2), _LIBRARY, (res[1], res[6], res[7])  # output, log-sum-exp, philox seed / offset


def _attention_backward(g: torch.Tensor, qkv: torch.Tensor, out: torch.Tensor, mode: int, saved, hq: int, hkv: int, cos, sin) -> torch.Tensor:
    """Packed ``dqkv`` for the output gradient ``g [B, S, hq, D]``, with RoPE's backward applied to its
    query and key heads (fused into the packing pass when the library returns three tensors)."""
    if mode == _NATIVE:
        from ..ops import attention_native as _n

        (lse,) = saved
        if _n._BACKWARD == "native":
            dqkv = _n.backward_packed(g.contiguous(), qkv, out.contiguous(), lse, hq, hkv)
            b, s, heads, hd = dqkv.shape
            _ext.get().rope_(dqkv.view(b * s, heads * hd), cos, sin, hq + hkv, hd, s, True)  # in place: this gradient is ours
            return dqkv
        dq, dk, dv = _n._library_backward(g.contiguous(), qkv, out, lse, hq, hkv, 1.0 / math.sqrt(qkv.shape[-1]))
    else:
        lse, seed, offset = saved
        q = qkv[:, :, :hq].transpose(1, 2)
        k = qkv[:, :, hq : hq + hkv].transpose(1, 2)
        v = qkv[:, :, hq + hkv :].transpose(1, 2)
        s = qkv.shape[1]
        dq, dk, dv = torch.ops.aten._scaled_dot_product_cudnn_attention_backward(
            g.transpose(1, 2), q, k, v, out.transpose(1, 2), lse, seed, offset, None, None, None, s, s, 0.0, True
        )
        dq, dk, dv = dq.transpose(1, 2), dk.transpose(1, 2), dv.transpose(1, 2)
    return _ext.get().pack_qkv_grad(dq, dk, dv, cos, sin)  # one pass: fused-QKV layout + RoPE backward


# ---------------------------------------------------------------------------------------
# forward / backward bodies shared by the three functions
# ---------------------------------------------------------------------------------------


def _attn_forward_body(blk, x: torch.Tensor):
    """``o = wo(attention(rope(wqkv(rmsnorm(x)))))`` (residual NOT added) and what the backward needs."""
    ext = _ext.get()
    b, s, d = x.shape
    hq, hkv, hd = blk.n_heads, blk.n_kv_heads, blk.head_dim
    cos, sin = blk._tables(x.device, s)
    h1, rstd1, _ = ext.rmsnorm_fwd(x, blk.norm1.weight, blk.norm1.eps, None)
    _stash_input(blk.wqkv, h1)
    qkv = _gemm.linear_forward(h1.view(b * s, d), blk.wqkv.weight)
    ext.rope_(qkv, cos, sin, hq + hkv, hd, s, False)
    qkv = qkv.view(b, s, hq + 2 * hkv, hd)
    a, mode, attn_saved = _attention_forward(qkv, hq, hkv)
    a = a.reshape(b, s, hq * hd)
    _stash_input(blk.wo, a)
    o = _gemm.linear_forward(a, blk.wo.weight)
    return o, mode, (rstd1, qkv, a, *attn_saved)


def _attn_backward_body(blk, x, mode, saved, dy: torch.Tensor) -> torch.Tensor:
    """Gradient w.r.t. ``x`` of ``x + o(x)`` given the gradient ``dy`` of that sum."""
    ext = _ext.get()
    rstd1, qkv, a = saved[:3]
    b, s, d = x.shape
    hq, hkv, hd = blk.n_heads, blk.n_kv_heads, blk.head_dim
    cos, sin = blk._tables(x.device, s)
    blk.wo._accumulate_grad_output(dy)
    d_a = _gemm.linear_input_grad(dy, blk.wo.weight)
    dqkv = _attention_backward(d_a.view(b, s, hq, hd), qkv, a.view(b, s, hq, hd), mode, saved[3:], hq, hkv, cos, sin)
    dqkv2 = dqkv.view(b * s, (hq + 2 * hkv) * hd)
    blk.wqkv._accumulate_grad_output(dqkv2)
    d_h1 = _gemm.linear_input_grad(dqkv2, blk.wqkv.weight)
    # norm backward + the residual branch's gradient in one pass; the gain's gradient goes
    # straight into its gradient buffer
    return ext.rmsnorm_bwd(d_h1.view(b, s, d), x, blk.norm1.weight, rstd1, _norm_grad_target(blk.norm1.weight), True, dy, None)


def _mlp_forward_body(blk, h2: torch.Tensor, x2: torch.Tensor):
    """``y = x2 + w_down(swiglu(w_gate_up(h2)))`` for the normalised ``h2`` of ``x2``."""
    ext = _ext.get()
    _stash_input(blk.w_gate_up, h2)
    gu = _gemm.linear_forward(h2, blk.w_gate_up.weight)
    act = ext.swiglu_fwd(gu)
    _stash_input(blk.w_down, act)
    dn = _gemm.linear_forward(act, blk.w_down.weight)
    return ext.residual_add(dn, x2), gu  # dn += x2, in place


def _mlp_backward_body(blk, x2, rstd2, gu, dy: torch.Tensor) -> torch.Tensor:
    ext = _ext.get()
    blk.w_down._accumulate_grad_output(dy)
    d_act = _gemm.linear_input_grad(dy, blk.w_down.weight)
    d_gu = ext.swiglu_bwd(d_act, gu)
    blk.w_gate_up._accumulate_grad_output(d_gu)
    d_h2 = _gemm.linear_input_grad(d_gu, blk.w_gate_up.weight)
    return ext.rmsnorm_bwd(d_h2, x2, blk.norm2.weight, rstd2, _norm_grad_target(blk.norm2.weight), True, dy, None)


# The weights are arguments of the functions (and get ``None`` gradients) so that the output
# requires grad even for an input that does not, and so that the partial backward replay
# (``zb_utils.partial_dx_recomputation``) finds these nodes right above the parameters.


class _AttentionHalf(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, blk, *weights):
        x = x.contiguous()
        o, mode, saved = _attn_forward_body(blk, x)
        y = _ext.get().residual_add(o, x)
        ctx.blk, ctx.mode = blk, mode
        ctx.save_for_backward(x, *saved)
        return y

    @staticmethod
    def backward(ctx, dy):
        x, *saved = ctx.saved_tensors
        dx = _attn_backward_body(ctx.blk, x, ctx.mode, saved, dy.contiguous())
        return (dx, None) + (None,) * 3


class _MLPHalf(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, blk, *weights):
        x = x.contiguous()
        h2, rstd2, _ = _ext.get().rmsnorm_fwd(x, blk.norm2.weight, blk.norm2.eps, None)
        y, gu = _mlp_forward_body(blk, h2, x)
        ctx.blk = blk
        ctx.save_for_backward(x, rstd2, gu)
        return y

    @staticmethod
    def backward(ctx, dy):
        x, rstd2, gu = ctx.saved_tensors
        dx = _mlp_backward_body(ctx.blk, x, rstd2, gu, dy.contiguous())
        return (dx, None) + (None,) * 3


class _DecoderLayer(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, blk, *weights):
        x = x.contiguous()
        o, mode, saved = _attn_forward_body(blk, x)
        h2, rstd2, x2 = _ext.get().rmsnorm_fwd(o, blk.norm2.weight, blk.norm2.eps, x)  # x2 = o + x, h2 = rmsnorm(x2)
        y, gu = _mlp_forward_body(blk, h2, x2)
        ctx.blk, ctx.mode = blk, mode
        ctx.save_for_backward(x, x2, rstd2, gu, *saved)
        return y

    @staticmethod
    def backward(ctx, dy):
        x, x2, rstd2, gu, *saved = ctx.saved_tensors
        dx2 = _mlp_backward_body(ctx.blk, x2, rstd2, gu, dy.contiguous())
        dx = _attn_backward_body(ctx.blk, x, ctx.mode, saved, dx2)
        return (dx, None) + (None,) * 6


# registered so that the partial backward replay treats these nodes like the per-linear ones
_FUSED_FUNCTIONS = (_AttentionHalf, _MLPHalf, _DecoderLayer)
for _fn in _FUSED_FUNCTIONS:
    LayerDW._dx_function_registry[_fn] = _fn


def attention_half(blk, x: torch.Tensor) -> torch.Tensor:
    """``blk`` provides ``norm1, wqkv, wo``, the head geometry and ``_tables``."""
    return _AttentionHalf.apply(x, blk, blk.norm1.weight, blk.wqkv.weight, blk.wo.weight)


def mlp_half(blk, x: torch.Tensor) -> torch.Tensor:
    """``blk`` provides ``norm2, w_gate_up, w_down``."""
    return _MLPHalf.apply(x, blk, blk.norm2.weight, blk.w_gate_up.weight, blk.w_down.weight)


def decoder_layer(blk, x: torch.Tensor) -> torch.Tensor:
    return _DecoderLayer.apply(x, blk, blk.norm1.weight, blk.wqkv.weight, blk.wo.weight, blk.norm2.weight, blk.w_gate_up.weight, blk.w_down.weight)
