"""Graph extraction: model → ``fx.GraphModule``.

Registered tracers (same keys as the reference, ``elf/partitioners/__init__.py:39-46``):

``fx``       ``torch.fx`` symbolic trace.  Split-backward layers (``LayerDW``) and any module
             with a truthy ``_elf_leaf`` attribute — how fused-kernel modules of this
             package declare themselves atomic — stay opaque ``call_module`` nodes.
``fx_safe``  like ``fx``, but sub-modules that cannot be traced are found bottom-up and
             their *classes* are made leaves, until the whole model traces.
``export``   ``torch.export.export(strict=False).module()``; last resort, because
             parameters become ``get_attr`` nodes that a partitioner may strand on a
             different stage than their user (``pin_get_attrs`` in the partition step
             repairs that).
``default``  ``fx``, then ``fx_safe``, then everything else that is registered.
"""

from __future__ import annotations

import logging
from typing import Iterable, List, Set

import torch
import torch.nn as nn
from torch.export import Dim

from ..registry import TRACERS, resolve
from ..zb_utils import LayerDWTracer

logger = logging.getLogger(__name__)

__all__ = [
    "trace",
    "extract_graph",
    "extract_graph_fx",
    "extract_graph_fx_safe",
    "extract_graph_export",
    "try_extract_graph",
    "PatchedTracer",
    "NonTraceableFinder",
    "filter_paths",
    "extract_module_by_name",
    "replace_module_inplace",
    "path_to_module",
    "get_shapes",
]


class PatchedTracer(LayerDWTracer):
    """``LayerDWTracer`` that also treats given classes and ``_elf_leaf`` modules as leaves."""

    def __init__(self, fx_leaf_modules: Iterable[type] = ()):
        super().__init__()
        self.fx_leaf_modules = list(fx_leaf_modules)

    def is_leaf_module(self, m: nn.Module, module_qualified_name: str) -> bool:
        if getattr(m, "_elf_leaf", False) or m.__class__ in self.fx_leaf_modules:
            return True
        return super().is_leaf_module(m, module_qualified_name)


def extract_graph_fx(model: nn.Module, *_sample) -> torch.fx.GraphModule:
    tracer = PatchedTracer()
    return torch.fx.GraphModule(model, tracer.trace(model))


def extract_graph_export(model: nn.Module, sample, run_decompositions: bool = True, use_dynamic_batch_size: bool = False):
    args = tuple(sample) if isinstance(sample, (list, tuple)) else (sample,)
    if use_dynamic_batch_size:
        shapes = tuple({0: Dim.DYNAMIC} for _ in args)
        program = torch.export.export(model, args=args, dynamic_shapes=shapes, strict=False)
        if run_decompositions:
            program = program.run_decompositions()
        return program.module()
    return torch.export.export(model, args=args, strict=False).module()


def filter_paths(paths: Iterable[str]) -> Set[str]:
    """Keep only the deepest paths: drop every path that is an ancestor of another one."""
    paths = set(paths)
    return {p for p in paths if not any(q.startswith(p + ".") for q in paths)}


def extract_module_by_name(root: nn.Module, name: str) -> nn.Module:
    cur = root
    for part in name.split("."):
        if hasattr(cur, part):
            cur = getattr(cur, part)
        elif isinstance(cur, (nn.ModuleList, nn.Sequential)) and part.isdigit():
            cur = cur[int(part)]
        else:
            raise ValueError(f"Module '{part}' not found in '{cur.__class__.__name__}'.")
    return cur


def replace_module_inplace(root: nn.Module, name: str, new_module: nn.Module) -> nn.Module:
    parent_name, _, leaf = name.rpartition(".")
    parent = extract_module_by_name(root, parent_name) if parent_name else root
    if not hasattr(parent, leaf):
        raise ValueError(f"Module '{leaf}' not found in '{parent.__class__.__name__}'.")
    old = getattr(parent, leaf)
    setattr(parent, leaf, new_module)
    return old


def path_to_module(root: nn.Module, module: nn.Module) -> str:
    for name, child in root.named_children():
        if child is module:
            return name
    raise NameError(f"Module {type(module)} is not a child of {type(root)}")


def get_shapes(x):
    if isinstance(x, torch.Tensor):
        return tuple(x.shape)
    if isinstance(x, (list, tuple)):
        return type(x)(get_shapes(v) for v in x)
    if isinstance(x, dict):
        return {k: get_shapes(v) for k, v in x.items()}
    return x


class NonTraceableFinder:
    """Finds the sub-modules of a model that a tracer cannot trace on their own."""

    def __init__(self, tracer: PatchedTracer):
        self.fx_tracer = tracer
        self.non_traceable_modules: List[str] = []
        self.non_traceable_leaf_modules: List[type] = []

    def get_non_traceable_modules(self, model: nn.Module, args=None) -> List[str]:
        bad = set()
        for name, module in model.named_modules():
            if name == "" or isinstance(module, nn.ModuleList):
                continue
            if self.fx_tracer.is_leaf_module(module, name):
                continue
            try:
                type(self.fx_tracer)(self.fx_tracer.fx_leaf_modules).trace(module)
            except Exception:
                bad.add(name)
        self.non_traceable_modules = sorted(bad)
        return self.non_traceable_modules

    def get_non_traceable_leaf_modules(self, model: nn.Module) -> List[type]:
        classes = {extract_module_by_name(model, p).__class__ for p in filter_paths(self.non_traceable_modules)}
        self.non_traceable_leaf_modules = sorted(classes, key=lambda c: c.__qualname__)
        return self.non_traceable_leaf_modules


def extract_graph_fx_safe(model: nn.Module, sample=None) -> torch.fx.GraphModule:
    leaves: List[type] = []
    for _ in range(64):  # each round adds at least one class; models have finitely many
        tracer = PatchedTracer(leaves)
        finder = NonTraceableFinder(tracer)
        finder.get_non_traceable_modules(model, sample)
        new = [c for c in finder.get_non_traceable_leaf_modules(model) if c not in leaves]
        if not new:
            return torch.fx.GraphModule(model, PatchedTracer(leaves).trace(model))
        leaves.extend(new)
    raise RuntimeError("fx_safe: leaf search did not converge")


def extract_graph(model, sample, mode: str = "fx"):
    if mode == "export":
        return extract_graph_export(model, sample)
    if mode == "fx":
        return extract_graph_fx(model)
    if mode == "fx_safe":
        return extract_graph_fx_safe(model, sample)
    raise ValueError(f"Unknown graph extraction mode: {mode}")


def try_extract_graph(model, sample):
    """``fx`` first, then ``fx_safe``, then the other registered tracers."""
    order = ["fx", "fx_safe"] + [k for k in TRACERS.available() if k not in ("default", "fx", "fx_safe")]
    errors = []
    for key in order:
        if key not in TRACERS:
            continue
        try:
            return TRACERS[key](model, sample)
        except Exception as exc:  # try the next, more permissive, tracer
            errors.append(f"{key}: {exc}")
            logger.info("Failed to extract graph with tracer %s. Trying next one.", key)
    raise RuntimeError("Failed to extract graph:\n" + "\n".join(errors))


def trace(model, sample, tracer="default") -> torch.fx.GraphModule:
    """Trace ``model`` with a tracer given by registry key or as a callable."""
    return resolve(tracer, TRACERS)(model, sample)
