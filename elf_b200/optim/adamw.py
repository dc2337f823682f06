"""Optimizers for the benchmark entry point.

``FusedAdamW``  bf16 parameters with fp32 master weights and fp32 Adam moments, updated by
one sm_100a kernel launch per flat buffer (``adamw_step`` in ``elf_b200/csrc/fused_ops.cu``).
It takes the place of the reference benchmark's ``MixedPrecisionOptimizer`` around
``torch.optim.AdamW`` (``benchmarks/run_transformer.py:46-121``), which copies every gradient
to an fp32 twin, steps, copies every weight back and synchronises the device twice.
On CPU tensors, or for dtypes other than bf16, the same class drives plain torch math.

``DummyOptimizer``  for ranks whose stages have no parameters (``:30-43``).
"""

from __future__ import annotations

import weakref
from typing import Iterable, List

import torch

from ..ops import _ext
from .flat import FlatGroup, flatten_parameters

__all__ = ["FusedAdamW", "DummyOptimizer", "MixedPrecisionOptimizer"]


class DummyOptimizer:
    def __init__(self, *args, **kwargs):
        self.param_groups: list = []

    def step(self):
        pass

    def zero_grad(self, set_to_none: bool = True):
        pass

    def state_dict(self):
        return {}

    def load_state_dict(self, state):
        pass


class FusedAdamW:
    def __init__(self, params: Iterable[torch.nn.Parameter], lr: float = 1e-3, betas=(0.9, 0.999), eps: float = 1e-8, weight_decay: float = 1e-2, grad_dtype=None):
        self.lr, self.betas, self.eps, self.weight_decay = lr, tuple(betas), eps, weight_decay
        self.step_count = 0
        self.groups: List[FlatGroup] = flatten_parameters(params, grad_dtype)
        self.master, self.exp_avg, self.exp_avg_sq = [], [], []
        for g in self.groups:
            self.master.append(g.flat_param.float())
            self.exp_avg.append(torch.zeros(g.numel, dtype=torch.float32, device=g.device))
            self.exp_avg_sq.append(torch.zeros(g.numel, dtype=torch.float32, device=g.device))
        self.param_groups = [{"params": [p for g in self.groups for p in g.params], "lr": lr}]
        for g in self.groups:  # lets whoever rewrites the parameters (a checkpoint load) find the fp32 copies
            g.optimizers = [o for o in getattr(g, "optimizers", []) if o() is not None] + [weakref.ref(self)]

    def resync_master(self) -> None:
        """Re-derive the fp32 master weights from the current parameter values.  Needed after
        anything other than this optimizer wrote the parameters (``load_state_dict`` on the
        model, ``Pipeline.load_checkpoint``): ``step`` rewrites the parameters from the master
        copy, so a stale master would silently undo the load.  ``Pipeline.load_checkpoint``
        calls this for every optimizer built over its parameters."""
        with torch.no_grad():
            for g, w in zip(self.groups, self.master):
                if w.data_ptr() != g.flat_param.data_ptr():
                    w.copy_(g.flat_param)

    def _kernel_ok(self, g: FlatGroup) -> bool:
        if g.device.type != "cuda" or g.dtype != torch.bfloat16:
            return False
        _ext.require_on_gpu()
        return g.grad_dtype in (torch.bfloat16, torch.float32)

    def zero_grad(self, set_to_none: bool = False) -> None:
        """Zero the flat gradient buffers; ``p.grad`` stays a view of them (``set_to_none``
        is accepted for API compatibility and ignored)."""
        for g in self.groups:
            g.zero_grad()

    @torch.no_grad()
    def step(self, grad_scale: float = 1.0) -> None:
        if self.groups and self.groups[0].device.type == "cuda":
            from ..ops import gemm

            gemm.raise_if_failed(self.groups[0].device)
        self.step_count += 1
        b1, b2 = self.betas
        lr = self.param_groups[0].get("lr", self.lr)
        for g, w, m, v in zip(self.groups, self.master, self.exp_avg, self.exp_avg_sq):
            g.gather_stray_grads()
            if self._kernel_ok(g):
                from ..ops import gemm

                _ext.get().adamw(g.flat_param, g.flat_grad, w, m, v, lr, b1, b2, self.eps, self.weight_decay, self.step_count, grad_scale,
                                 gemm.status(g.device))
                gemm.snapshot_status_async(g.device)
                continue
            grad = g.flat_grad.float() * grad_scale
            m.mul_(b1).add_(grad, alpha=1 - b1)
            v.mul_(b2).addcmul_(grad, grad, value=1 - b2)
            bc1, bc2 = 1 - b1**self.step_count, 1 - b2**self.step_count
            w.mul_(1 - lr * self.weight_decay).addcdiv_(m / bc1, (v / bc2).sqrt_().add_(self.eps), value=-lr)
            g.flat_param.copy_(w)

    def state_dict(self) -> dict:
        return {
            "step": self.step_count,
            "lr": self.lr,
            "betas": self.betas,
            "eps": self.eps,
            "weight_decay": self.weight_decay,
            "master": [t.cpu() for t in self.master],
            "exp_avg": [t.cpu() for t in self.exp_avg],
            "exp_avg_sq": [t.cpu() for t in self.exp_avg_sq],
        }

    def load_state_dict(self, state: dict) -> None:
        self.step_count = int(state["step"])
        for dst_list, key in ((self.master, "master"), (self.exp_avg, "exp_avg"), (self.exp_avg_sq, "exp_avg_sq")):
            for dst, src in zip(dst_list, state[key]):
                dst.copy_(src)
        for g, w in zip(self.groups, self.master):
            g.flat_param.copy_(w)


class MixedPrecisionOptimizer:
    """Generic wrapper kept for parity with the reference CLI: runs any torch optimizer on
    ``opt_dtype`` copies of the parameters living on ``opt_device``."""

    def __init__(self, optimizer_cls, params, dtype, opt_dtype, opt_device, **kwargs):
        params = [p for p in params if p.requires_grad]
        self.opt_device = torch.device(opt_device)
        self.need_master = dtype != opt_dtype or (params and self.opt_device.type != params[0].device.type)
        if self.need_master:
            self.pairs = [(p, p.detach().clone().to(opt_dtype).to(self.opt_device).requires_grad_(True)) for p in params]
            self.optimizer = optimizer_cls([m for _, m in self.pairs], **kwargs)
        else:
            self.pairs = []
            self.optimizer = optimizer_cls(params, **kwargs)

    def zero_grad(self, set_to_none: bool = False):
        for p, m in self.pairs:
            if m.grad is not None:
                m.grad.zero_()
            if p.grad is not None:
                p.grad.zero_()
        if not self.need_master:
            self.optimizer.zero_grad(set_to_none=set_to_none)

    def step(self):
        if not self.need_master:
            return self.optimizer.step()
        for p, m in self.pairs:
            if p.grad is not None:
                if m.grad is None:
                    m.grad = torch.empty_like(m, pin_memory=self.opt_device.type == "cpu" and torch.cuda.is_available())
                m.grad.copy_(p.grad, non_blocking=True)
        if torch.cuda.is_available():
            torch.cuda.current_stream().synchronize()
        self.optimizer.step()
        for p, m in self.pairs:
            p.data.copy_(m.data, non_blocking=True)

    def state_dict(self):
        return self.optimizer.state_dict()

    def load_state_dict(self, state):
        self.optimizer.load_state_dict(state)

    def __getattr__(self, name):
        return getattr(self.optimizer, name)
