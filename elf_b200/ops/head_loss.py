"""LM head + cross entropy without ever holding the logits (vocabulary processed in chunks).

The plain path projects the final hidden states onto the whole vocabulary (1 GB of bf16
logits per 4096-token micro-batch at a 128 k vocabulary), runs the cross-entropy kernels over
that buffer and turns it into the gradient in place.  ``chunked_head_loss`` walks the
vocabulary in column chunks instead:

forward   per chunk: ``logits_c = h · W_cᵀ`` (tcgen05 GEMM) → fold into the running row maximum,
          sum of exponentials and target logit → drop the chunk; ``loss = Σ (lse − target logit)``
backward  per chunk: recompute ``logits_c``, turn it into ``(softmax − onehot) · scale`` in place,
          ``dh += dlogits_c · W_c`` (fp32 accumulator) and ``dW_c += dlogits_cᵀ · h`` straight into
          the weight's gradient buffer

so the largest temporary is one chunk (``rows × chunk`` bf16).  The price is one more GEMM
over the vocabulary (the recomputation), about a third of the head's FLOPs; it buys
``rows × vocab × 2`` bytes per micro-batch in flight on the last stage, which is what a tight
``memory_budget`` wants.  It replaces the reference model zoo's fp32 ``F.cross_entropy`` over
full logits (``benchmarks/models/simple.py:512-524``).

Both the input gradient and the weight gradient are produced in the backward of the loss (the
weight gradient does not wait for a W pass: deferring it would mean keeping or recomputing the
vocabulary-sized gradient a second time).
"""

from __future__ import annotations

from typing import Optional

import torch
import torch.nn.functional as F

from . import _ext
from . import fused as _f
from . import gemm as _gemm

__all__ = ["chunked_head_loss", "ChunkedHeadLoss", "default_chunk"]


def default_chunk(vocab: int, target: int = 16384) -> int:
    """Largest divisor-free choice is not needed: the last chunk may be narrower.  Chunks are
    multiples of 256 columns (whole GEMM tiles)."""
    return max(256, min(vocab, (target + 255) // 256 * 256))


def _grad_target(w: torch.Tensor) -> torch.Tensor:
    target = getattr(w, "main_grad", None)
    if target is None:
        if w.grad is None:
            w.grad = torch.zeros_like(w)
        target = w.grad
    return target


class _ChunkedHeadLoss(torch.autograd.Function):
    @staticmethod
    def forward(ctx, h, weight, targets, chunk, scale, ignore_index):
        ext = _ext.get()
        h2 = h.reshape(-1, h.shape[-1])
        if not h2.is_contiguous():
            h2 = h2.contiguous()
        rows, vocab = h2.shape[0], weight.shape[0]
        t = targets.reshape(-1).contiguous()
        run_max = torch.empty(rows, dtype=torch.float32, device=h.device)
        run_sum = torch.empty_like(run_max)
        tgt = torch.empty_like(run_max)
        for c0 in range(0, vocab, chunk):
            c1 = min(vocab, c0 + chunk)
            logits = _gemm.matmul_nt(h2, weight[c0:c1])
            ext.ce_chunk_stats(logits, t, run_max, run_sum, tgt, c0, c0 == 0)
            del logits
        lse = run_max + torch.log(run_sum)
        valid = (t != ignore_index) & (t >= 0) & (t < vocab)
        loss = torch.where(valid, lse - tgt, torch.zeros_like(lse)).sum() * scale
        ctx.save_for_backward(h2, weight, t, lse)
        ctx.chunk, ctx.scale, ctx.ignore_index, ctx.shape = chunk, scale, ignore_index, h.shape
        return loss

    @staticmethod
    def backward(ctx, g):
        ext = _ext.get()
        h2, weight, t, lse = ctx.saved_tensors
        rows, vocab = h2.shape[0], weight.shape[0]
        gs = g.detach().to(torch.float32).reshape(1).contiguous()
        dh = torch.zeros(rows, h2.shape[1], dtype=torch.float32, device=h2.device)
        wgrad = _grad_target(weight)
        status = _gemm.status(h2.device)
        for c0 in range(0, vocab, ctx.chunk):
            c1 = min(vocab, c0 + ctx.chunk)
            d = _gemm.matmul_nt(h2, weight[c0:c1])  # the chunk's logits again
            ext.ce_chunk_grad(d, t, lse, gs, ctx.scale, c0, vocab, ctx.ignore_index)
            # dh (fp32) += d · W_c : A = d K-major, B = W_c MN-major
            ext.gemm(d, weight[c0:c1], dh, None, False, True, True, 1.0, status, _gemm._VARIANT, False)
            # dW_c += dᵀ · h : both operands MN-major, accumulated in the epilogue
            _gemm.linear_weight_grad(d, h2, out=wgrad[c0:c1])
            del d
        return dh.to(h2.dtype).view(ctx.shape), None, None, None, None, None


def chunked_head_loss(h: torch.Tensor, weight: torch.Tensor, target: torch.Tensor, reduction: str = "mean", ignore_index: int = -100, chunk: Optional[int] = None) -> torch.Tensor:
    """Cross entropy of ``h · weightᵀ`` against ``target`` with the vocabulary in chunks.

    ``h [..., d]`` are the (already normalised) final hidden states, ``weight [vocab, d]`` the
    head's matrix (a parameter: its gradient is accumulated into ``weight.grad`` during the
    backward).  On CPU, or for dtypes the kernels do not handle, the plain formula is used."""
    vocab = weight.shape[0]
    flat_t = target.reshape(-1)
    if _f.kernels_apply(h) and weight.is_cuda and weight.dtype == h.dtype and reduction in ("sum", "mean") and h.shape[-1] % 8 == 0 and vocab % 8 == 0:
        if reduction == "mean":
            valid = (flat_t != ignore_index).sum().clamp_min(1).item() if ignore_index >= 0 else flat_t.numel()
            scale = 1.0 / max(valid, 1)
        else:
            scale = 1.0
        return _ChunkedHeadLoss.apply(h, weight, flat_t, int(chunk or default_chunk(vocab)), scale, ignore_index)
    logits = F.linear(h, weight)
    return F.cross_entropy(logits.float().reshape(-1, vocab), flat_t, reduction=reduction, ignore_index=ignore_index)


class ChunkedHeadLoss:
    """Loss function for a pipeline whose last stage ends with a head in *deferred* mode
    (``LlamaHead(cfg, fused_loss=True)`` returns the normalised hidden states instead of logits):
    ``loss_fn = ChunkedHeadLoss(head)`` then ``pipe(batch, target, loss_fn)``.  The head's matrix
    stays a parameter of the stage (optimizer, checkpoints and the data-parallel exchange see it);
    this object only reads it and adds to its gradient."""

    def __init__(self, head, chunk: Optional[int] = None, ignore_index: int = -100):
        self.head, self.chunk, self.ignore_index = head, chunk, ignore_index

    def __call__(self, hidden, target, reduction: str = "mean"):
        return chunked_head_loss(hidden, self.head.out.weight, target, reduction, self.ignore_index, self.chunk)
