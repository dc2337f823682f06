"""Flat parameter / gradient storage.

Re-homes a list of parameters into one contiguous buffer per dtype and gives every
parameter a gradient that is a view of one contiguous gradient buffer.  One fused kernel
can then update all parameters, and the data-parallel gradient exchange moves one buffer
per stage instead of one message per tensor (the reference all-reduces tensor by tensor,
``elf/execution/block.py:506-516``).
"""

from __future__ import annotations

from typing import Dict, Iterable, List, Tuple

import torch

__all__ = ["FlatGroup", "flatten_parameters"]

_ALIGN = 128  # elements; keeps every view 256-byte aligned for 16-bit types


class FlatGroup:
    """Parameters of one dtype on one device sharing ``flat_param`` and ``flat_grad``."""

    def __init__(self, params: List[torch.nn.Parameter], grad_dtype=None):
        assert params, "empty group"
        self.params = params
        p0 = params[0]
        self.dtype, self.device = p0.dtype, p0.device
        self.grad_dtype = grad_dtype or p0.dtype
        self.offsets: List[int] = []
        total = 0
        for p in params:
            self.offsets.append(total)
            total += (p.numel() + _ALIGN - 1) // _ALIGN * _ALIGN
        self.numel = total
        self.flat_param = torch.zeros(total, dtype=self.dtype, device=self.device)
        for p, off in zip(params, self.offsets):  # one tensor at a time: peak = +1 tensor
            view = self.flat_param[off : off + p.numel()].view(p.shape)
            view.copy_(p.data)
            p.data = view
        self.flat_grad = torch.zeros(total, dtype=self.grad_dtype, device=self.device)
        self.attach_grads()
        for p in params:
            p._elf_flat_group = self  # lets a later flatten (the optimizer's) adopt this group

    def grad_view(self, i: int) -> torch.Tensor:
        p, off = self.params[i], self.offsets[i]
        return self.flat_grad[off : off + p.numel()].view(p.shape)

    def attach_grads(self) -> None:
        """Point every ``p.grad`` at its slice of ``flat_grad`` (only possible when the
        gradient dtype equals the parameter dtype; otherwise slices are exposed as
        ``p.main_grad``)."""
        for i, p in enumerate(self.params):
            if self.grad_dtype == p.dtype:
                p.grad = self.grad_view(i)
            else:
                p.main_grad = self.grad_view(i)

    def gather_stray_grads(self) -> None:
        """Fold gradients that were re-allocated outside the flat buffer (for example after
        ``zero_grad(set_to_none=True)``) back into it."""
        for i, p in enumerate(self.params):
            if self.grad_dtype != p.dtype:
                if p.grad is not None:
                    self.grad_view(i).add_(p.grad)
                    p.grad = None
                continue
            view = self.grad_view(i)
            if p.grad is None:
                p.grad = view
            elif p.grad.data_ptr() != view.data_ptr():
                view.copy_(p.grad)
                p.grad = view

    def zero_grad(self) -> None:
        self.flat_grad.zero_()
        self.attach_grads()


def flatten_parameters(params: Iterable[torch.nn.Parameter], grad_dtype=None) -> List[FlatGroup]:
    """Groups already built for (all of) these parameters - e.g. by the data-parallel gradient
    exchange - are reused, so one flat buffer serves both the exchange and the optimizer."""
    buckets: Dict[Tuple[torch.dtype, torch.device], List[torch.nn.Parameter]] = {}
    adopted: Dict[int, FlatGroup] = {}
    seen = set()
    for p in params:
        if not p.requires_grad or id(p) in seen or p.is_meta:
            continue
        seen.add(id(p))
        existing = getattr(p, "_elf_flat_group", None)
        if existing is not None:
            adopted[id(existing)] = existing
            continue
        buckets.setdefault((p.dtype, p.device), []).append(p)
    for g in adopted.values():
        missing = [q for q in g.params if id(q) not in seen]
        if missing:
            raise ValueError("a flat parameter group can only be adopted whole; pass all of its parameters")
    return list(adopted.values()) + [FlatGroup(ps, grad_dtype) for ps in buckets.values()]
