"""Split backward (Zero-Bubble B / W passes) for parameterised layers.

A ``LayerDW`` layer computes, during autograd's backward, only the gradient w.r.t. its
*input* (the B pass) and stashes what the weight gradient needs — the layer input seen in
the forward and the output-gradient seen in the backward — per micro-batch.  A later
``layer.backward(mb_id)`` call (the W pass) turns one stashed pair into ``weight.grad``.
User-visible protocol and names follow the reference (``elf/zb_utils.py``): ``ctx`` with the
``"input"``/``"grad_output"`` queues, ``last_input``/``last_grad_output`` staging slots,
``move_last_computed``, ``delete``, ``is_empty``, ``clear``, ``offload_last``,
``replace_layer_with_layer_dw``, ``LayerDWTracer`` and ``partial_dx_recomputation``.

On a CUDA device with bf16 operands the three GEMMs of ``LinearDW``
(``Y = X·Wᵀ``, ``dX = dY·W``, ``dW += dYᵀ·X``) run on this package's sm_100a tcgen05
kernels (``elf_b200.ops.gemm``); the weight-gradient kernel accumulates into the existing
``weight.grad`` inside its epilogue, so there is no separate ``grad.add_`` pass as in the
reference (``elf/zb_utils.py:241-252``).  Everything else falls back to torch ops.
"""

from __future__ import annotations

from typing import Dict, Iterable, List, Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

from .ops import gemm as _gemm

__all__ = [
    "LayerDW",
    "LinearDX",
    "LinearDW",
    "Conv1dDX",
    "Conv1dDW",
    "MappingDW",
    "replace_layer_with_layer_dw",
    "replace_linear_with_linear_dw",
    "LayerDWTracer",
    "partial_dx_recomputation",
    "in_partial_replay",
]


def _flat2d(t: torch.Tensor) -> torch.Tensor:
    return t if t.dim() == 2 else t.reshape(-1, t.size(-1))


class LayerDW:
    """Mixin (list it *before* the ``nn.Module`` base) adding the W-pass stash."""

    _dx_function_registry: Dict[type, type] = {}

    def __init__(self, *args, **kwargs):
        # The shell is built on ``meta``: its tensors are replaced by the wrapped layer's.
        with torch.device("meta"):
            super().__init__(*args, **kwargs)
        self.ctx: Dict[str, List[Optional[torch.Tensor]]] = {"input": [], "grad_output": []}
        self.last_input: Optional[torch.Tensor] = None
        self.last_grad_output: Optional[torch.Tensor] = None

    @classmethod
    def register_dx_function(cls, dx_class):
        """Declare ``dx_class`` (an ``autograd.Function``) as this layer type's B pass."""
        LayerDW._dx_function_registry[cls] = dx_class
        return dx_class

    # -- W pass -------------------------------------------------------------
    def backward(self, mb_id: int):  # pragma: no cover - interface
        raise NotImplementedError("Subclasses must implement backward()")

    def _take(self, mb_id: int):
        """Pop the (input, grad_output) pair of ``mb_id``."""
        try:
            x, g = self.ctx["input"][mb_id], self.ctx["grad_output"][mb_id]
        except IndexError:
            x = g = None
        if x is None or g is None:
            raise ValueError(f"W pass of micro-batch {mb_id}: stash is incomplete (input={x is not None}, grad={g is not None})")
        self.ctx["input"][mb_id] = None
        self.ctx["grad_output"][mb_id] = None
        return x, g

    # -- stash bookkeeping ----------------------------------------------------
    def clear(self) -> None:
        self.ctx["input"].clear()
        self.ctx["grad_output"].clear()
        self.last_input = None
        self.last_grad_output = None

    def is_empty(self, queue: str) -> bool:
        return all(v is None for v in self.ctx[queue])

    def _state(self) -> str:
        count = lambda q: sum(v is not None for v in self.ctx[q])
        return f"({count('input')},{count('grad_output')})"

    def _store_input(self, input: torch.Tensor) -> None:
        stash = input.detach()
        # A tensor with no grad_fn is a stage input: checkpoint recomputation will not
        # regenerate it, so remat must not drop it.
        stash.is_model_input = input.grad_fn is None
        self.last_input = stash

    def _accumulate_grad_output(self, grad_output: torch.Tensor) -> None:
        # A layer applied several times in one forward receives several output-grads.
        prev = getattr(self, "last_grad_output", None)
        self.last_grad_output = grad_output if prev is None else prev + grad_output

    def set(self, queue: str, idx: int, value) -> None:
        slots = self.ctx[queue]
        if len(slots) <= idx:
            slots.extend([None] * (idx + 1 - len(slots)))
        if slots[idx] is not None:
            raise ValueError(f"{queue} at index {idx} already set")
        slots[idx] = value

    def delete(self, queue: str, idx: int) -> None:
        slots = self.ctx[queue]
        if idx >= len(slots) or slots[idx] is None:
            raise ValueError(f"{queue} at index {idx} not set")
        slots[idx] = None

    def move_last_computed(self, queue: str, idx: int) -> None:
        """File the staged ``last_<queue>`` tensor under micro-batch ``idx`` (no-op if the
        layer did not take part in the last pass)."""
        staged = getattr(self, f"last_{queue}", None)
        if staged is None:
            return
        self.set(queue, idx, staged)
        setattr(self, f"last_{queue}", None)

    def offload_last(self, idx: int, to="cpu") -> None:
        """Move the stashed pair of micro-batch ``idx`` to ``to`` (asynchronously when the
        destination is pinned host memory); ``backward`` brings it back."""
        with torch.no_grad():
            for q in ("input", "grad_output"):
                t = self.ctx[q][idx] if idx < len(self.ctx[q]) else None
                if t is not None:
                    self.ctx[q][idx] = t.to(to, non_blocking=True)


# ---------------------------------------------------------------------------------------
# Linear
# ---------------------------------------------------------------------------------------


class LinearDX(torch.autograd.Function):
    """``y = x Wᵀ + b`` whose backward returns only ``dx = dy W``."""

    @staticmethod
    def forward(ctx, input, weight, bias, linear):
        # weight/bias are arguments so the output requires grad even if ``input`` does not
        ctx.linear = linear
        linear._store_input(input)
        # saved (although unused here) so that torch.utils.checkpoint recomputes it
        ctx.save_for_backward(input.detach())
        if _gemm.usable(input, weight):
            return _gemm.linear_forward(input, weight, bias)
        return F.linear(input, weight, bias)

    @staticmethod
    def backward(ctx, grad_output):
        linear = ctx.linear
        linear._accumulate_grad_output(grad_output)
        weight = linear.weight
        if grad_output.is_complex():
            weight = weight.conj()  # Wirtinger: dL/dx = dL/dy · conj(W)
        elif _gemm.usable(grad_output, weight):
            return _gemm.linear_input_grad(grad_output, weight), None, None, None
        return torch.matmul(grad_output, weight), None, None, None


class LinearDW(LayerDW, nn.Linear):
    """Drop-in for ``nn.Linear`` sharing the wrapped layer's parameters."""

    def __init__(self, linear: nn.Linear, *args, **kwargs):
        super().__init__(linear.in_features, linear.out_features, linear.bias is not None, *args, **kwargs)
        self.weight = linear.weight
        if linear.bias is not None:
            self.bias = linear.bias

    def forward(self, x, *args, **kwargs):
        return LinearDX.apply(x, self.weight, self.bias, self)

    def backward(self, mb_id: int) -> None:
        x, g = self._take(mb_id)
        dev = self.weight.device
        if x.device != dev:
            x = x.to(dev, non_blocking=True)
        if g.device != dev:
            g = g.to(dev, non_blocking=True)
        g2, x2 = _flat2d(g), _flat2d(x)
        with torch.no_grad():
            if not g2.is_complex() and _gemm.usable(g2, self.weight) and _gemm.grad_buffer_ok(self.weight):
                # dW (+)= dYᵀ·X with the accumulation fused in the kernel epilogue.  On the
                # step's last W pass of a data-parallel run the epilogue also pushes the
                # finished gradient to the other replicas (elf_b200.parallel.dp_sync).
                push = None
                plan = getattr(self, "_push", None)
                if plan is not None and getattr(self, "_final_pass", False) and self.weight.grad is not None and self.weight.grad.dtype == self.weight.dtype:
                    push = plan.target()
                self.weight.grad = _gemm.linear_weight_grad(g2, x2, out=self.weight.grad, push=push)
            else:
                dw = torch.mm(g2.t(), x2.conj() if g2.is_complex() else x2)
                if self.weight.grad is None:
                    self.weight.grad = dw
                else:
                    self.weight.grad.add_(dw)
            if self.bias is not None:
                db = g2.sum(0)
                if self.bias.grad is None:
                    self.bias.grad = db.to(self.bias.dtype)
                else:
                    self.bias.grad.add_(db)


LinearDW.register_dx_function(LinearDX)


# ---------------------------------------------------------------------------------------
# Conv1d (torch/cuDNN ops; no sm_100a kernel: not on any benchmarked path)
# ---------------------------------------------------------------------------------------


def _conv1d_geometry(conv: nn.Conv1d, l_in: int, l_out: int):
    one = lambda v: v[0] if isinstance(v, (tuple, list)) else v
    stride, dilation = one(conv.stride), one(conv.dilation)
    k = conv.weight.shape[2]
    padding = conv.padding
    if isinstance(padding, str):
        if padding == "same":
            padding = max(0, (l_out - 1) * stride + dilation * (k - 1) + 1 - l_in) // 2
        else:  # "valid"
            padding = 0
    return stride, one(padding), dilation, k


class Conv1dDX(torch.autograd.Function):
    @staticmethod
    def forward(ctx, input, weight, bias, conv1d):
        ctx.conv1d = conv1d
        conv1d._store_input(input)
        ctx.save_for_backward(input.detach())
        return F.conv1d(input, weight, bias, conv1d.stride, conv1d.padding, conv1d.dilation, conv1d.groups)

    @staticmethod
    def backward(ctx, grad_output):
        conv = ctx.conv1d
        conv._accumulate_grad_output(grad_output)
        (x,) = ctx.saved_tensors
        with torch.no_grad():
            stride, padding, dilation, k = _conv1d_geometry(conv, x.shape[2], grad_output.shape[2])
            out_pad = x.shape[2] - ((grad_output.shape[2] - 1) * stride - 2 * padding + dilation * (k - 1) + 1)
            w = conv.weight.conj() if grad_output.is_complex() else conv.weight
            dx = F.conv_transpose1d(grad_output, w, None, stride, padding, out_pad, conv.groups, dilation)
        return dx, None, None, None


class Conv1dDW(LayerDW, nn.Conv1d):
    def __init__(self, conv1d: nn.Conv1d, *args, **kwargs):
        super().__init__(
            conv1d.in_channels,
            conv1d.out_channels,
            conv1d.kernel_size,
            *args,
            stride=conv1d.stride,
            padding=conv1d.padding,
            dilation=conv1d.dilation,
            groups=conv1d.groups,
            bias=conv1d.bias is not None,
            **kwargs,
        )
        self.weight = conv1d.weight
        if conv1d.bias is not None:
            self.bias = conv1d.bias

    def forward(self, x, *args, **kwargs):
        return Conv1dDX.apply(x, self.weight, self.bias, self)

    def _weight_grad_complex(self, x, g, stride, padding, dilation, k):
        """Complex dW by explicit correlation with the conjugated input (the native
        conv-backward kernels reject complex dtypes)."""
        n, l_out = x.shape[0], g.shape[2]
        xp = F.pad(x, (padding, padding)) if padding > 0 else x
        sb, sc, sl = xp.stride()
        patches = xp.as_strided((n, self.in_channels, k, l_out), (sb, sc, dilation * sl, stride * sl))
        cin_g, cout_g = self.in_channels // self.groups, self.out_channels // self.groups
        pg = patches.reshape(n, self.groups, cin_g, k, l_out)
        gg = g.reshape(n, self.groups, cout_g, l_out)
        dw = torch.einsum("ngol,ngikl->goik", gg, pg.conj())
        return dw.reshape(self.out_channels, cin_g, k)

    def backward(self, mb_id: int) -> None:
        x, g = self._take(mb_id)
        with torch.no_grad():
            stride, padding, dilation, k = _conv1d_geometry(self, x.shape[2], g.shape[2])
            if x.is_complex():
                dw = self._weight_grad_complex(x, g, stride, padding, dilation, k)
            else:
                dw = torch.nn.grad.conv1d_weight(x, self.weight.shape, g, [stride], [padding], [dilation], self.groups)
            dw = dw.to(self.weight.device, non_blocking=True)
            if self.weight.grad is None:
                self.weight.grad = dw
            else:
                self.weight.grad.add_(dw)
            if self.bias is not None:
                db = g.sum(dim=(0, 2)).to(self.bias.device, non_blocking=True)
                if self.bias.grad is None:
                    self.bias.grad = db
                else:
                    self.bias.grad.add_(db)


Conv1dDW.register_dx_function(Conv1dDX)


# ---------------------------------------------------------------------------------------
# model surgery
# ---------------------------------------------------------------------------------------

MappingDW = {nn.Linear: LinearDW, nn.Conv1d: Conv1dDW}


def _swap_children(model: nn.Module, make) -> None:
    for name, module in list(model.named_modules()):
        replacement = make(module)
        if replacement is None or name == "":
            continue
        parent_name, _, child = name.rpartition(".")
        parent = model.get_submodule(parent_name) if parent_name else model
        setattr(parent, child, replacement)


def replace_layer_with_layer_dw(model: nn.Module, only: Optional[Iterable[type]] = None) -> nn.Module:
    """In place: swap every layer whose exact type has a split-backward twin
    (``MappingDW``), optionally restricted to the types in ``only``."""
    only = None if only is None else set(only)

    def make(m):
        t = type(m)
        if t in MappingDW and not isinstance(m, LayerDW) and (only is None or t in only):
            return MappingDW[t](m)
        return None

    _swap_children(model, make)
    return model


def replace_linear_with_linear_dw(model: nn.Module, device=None) -> nn.Module:
    """Deprecated spelling kept for old scripts: swaps ``nn.Linear`` (and subclasses) only.
    ``device`` is ignored: the twin adopts the original layer's tensors wherever they are."""

    def make(m):
        if isinstance(m, nn.Linear) and not isinstance(m, LayerDW):
            return LinearDW(m)
        return None

    _swap_children(model, make)
    return model


class LayerDWTracer(torch.fx.Tracer):
    """fx tracer that never looks inside a ``LayerDW`` layer."""

    def is_leaf_module(self, m: nn.Module, module_qualified_name: str) -> bool:
        return isinstance(m, LayerDW) or super().is_leaf_module(m, module_qualified_name)


# ---------------------------------------------------------------------------------------
# partial backward replay (B → W recompute of output-grads)
# ---------------------------------------------------------------------------------------


_replay_depth = 0


def in_partial_replay() -> bool:
    """True while ``partial_dx_recomputation`` runs: a backward node that also accumulates
    parameter gradients as a side effect (a fused layer's norm gains) must skip that part, the
    first backward has already added them."""
    return _replay_depth > 0


def _dx_node_names() -> set:
    return {f"{fn.__name__}Backward" for fn in LayerDW._dx_function_registry.values()}


def _leaves_below_dx(root) -> list:
    """AccumulateGrad leaves of the autograd graph under ``root`` whose *direct* producer
    is a split-backward node.  Differentiating w.r.t. exactly these leaves makes autograd
    run every ``*DX.backward`` (refilling the output-grad stashes) and nothing deeper."""
    names = _dx_node_names()
    seen = set()
    leaves = []
    stack = [(root, False)]
    while stack:  # iterative: a recursive closure would keep grad_fn objects alive
        node, parent_is_dx = stack.pop()
        if node is None or node in seen:
            continue
        seen.add(node)
        if not node.next_functions:
            if parent_is_dx and hasattr(node, "variable"):
                leaves.append(node)
            continue
        is_dx = type(node).__name__ in names
        for nxt, _ in node.next_functions:
            if nxt is not None and nxt not in seen:
                stack.append((nxt, is_dx))
    return [torch.autograd.graph.get_gradient_edge(n.variable) for n in leaves]


def partial_dx_recomputation(outputs, grad_outputs=None, retain_graph: bool = False) -> None:
    """Run the smallest backward that refills the ``grad_output`` stash of every
    ``LayerDW`` layer under ``outputs``."""
    global _replay_depth
    _replay_depth += 1
    try:
        _partial_dx_recomputation(outputs, grad_outputs, retain_graph)
    finally:
        _replay_depth -= 1


def _partial_dx_recomputation(outputs, grad_outputs, retain_graph: bool) -> None:
    if grad_outputs is None:
        assert outputs.numel() == 1, "Implicit gradient outputs are only supported for scalar outputs"
        grad_outputs = torch.ones_like(outputs)
    if isinstance(outputs, (list, tuple)):
        # several outputs of one stage: one traversal, so that nodes they share run their backward once
        seen, edges = set(), []
        for o in outputs:
            for e in _leaves_below_dx(o.grad_fn):
                if e.node not in seen:
                    seen.add(e.node)
                    edges.append(e)
        if edges:
            torch.autograd.grad(list(outputs), inputs=edges, grad_outputs=list(grad_outputs), allow_unused=True, retain_graph=retain_graph)
        return
    edges = _leaves_below_dx(outputs.grad_fn)
    if edges:
        torch.autograd.grad(outputs, inputs=edges, grad_outputs=grad_outputs, allow_unused=True, retain_graph=retain_graph)
