"""Partitioning helpers: signatures (re-exported), graph clean-ups, DOT export."""

from __future__ import annotations

import re
import shutil
import subprocess
import sys
from typing import List, Optional, TextIO

import torch
import torch.fx as fx

from .signature import (  # noqa: F401  (public re-exports)
    Signature,
    get_sources_targets_sequential,
    remove_dupes,
    sequential_signatures,
    signatures_from_sources_targets,
)

__all__ = [
    "remove_inplace_leaves",
    "sequential_signatures",
    "Signature",
    "signatures_from_sources_targets",
    "prune_graph",
    "partition_to_dot",
    "export_partition_to_image",
]

_ALIAS_RETURN = re.compile(r"-> \(?Tensor\([a-z]")


def _returns_alias(target) -> bool:
    """True when the op's schema says its result aliases an argument (a view)."""
    schema = getattr(target, "_schema", None)
    return schema is not None and bool(_ALIAS_RETURN.search(str(schema)))


def _base_name(target) -> Optional[str]:
    name = getattr(target, "__name__", None)
    return None if name is None else name.split(".")[0]


def _is_inplace(target) -> bool:
    schema = getattr(target, "_schema", None)
    if schema is not None:
        try:
            return bool(schema.is_mutable)
        except AttributeError:
            pass
    base = _base_name(target)
    return base is not None and base.endswith("_") and not base.endswith("__")


def _out_of_place(target):
    base = _base_name(target)
    if base is None or not base.endswith("_"):
        raise ValueError(f"{target} does not look like an in-place op")
    plain = base[:-1]
    overload = getattr(target, "_overloadname", None)
    if overload is not None:
        try:
            return getattr(getattr(torch.ops.aten, plain), overload)
        except AttributeError as exc:
            raise ValueError(f"no ATen op aten.{plain}.{overload}") from exc
    for home in (torch, torch.nn.functional):
        if hasattr(home, plain):
            return getattr(home, plain)
    raise ValueError(f"Could not find out-of-place equivalent for {target}")


def remove_inplace_leaves(module: fx.GraphModule) -> fx.GraphModule:
    """Make in-place ops that act directly on stage inputs (or on views of them)
    out-of-place.  A stage's inputs are autograd leaves that require grad; PyTorch forbids
    mutating those in place, which would break every stage whose first op is e.g.
    ``relu_`` or ``nn.ReLU(inplace=True)`` (reference ``elf/partitioners/utils.py:149-302``)."""
    g = module.graph
    owner = g.owning_module
    view_methods = {"view", "reshape", "transpose", "permute", "squeeze", "unsqueeze", "flatten", "t", "contiguous", "narrow", "select", "expand", "view_as", "__getitem__"}
    # tensors that share storage with a stage input: the inputs and (chains of) views of them
    aliases = {nd for nd in g.nodes if nd.op == "placeholder"}
    for node in g.nodes:  # topological order: one pass reaches the fixed point
        if node.op in ("placeholder", "output") or not node.all_input_nodes:
            continue
        first = node.args[0] if node.args and isinstance(node.args[0], fx.Node) else None
        touches_input = first in aliases if first is not None else False
        if not touches_input:
            continue
        if node.op == "call_function":
            if _is_inplace(node.target):
                node.target = _out_of_place(node.target)  # result is a fresh tensor
            elif node.kwargs.get("inplace", False):
                node.kwargs = {**node.kwargs, "inplace": False}
            elif _returns_alias(node.target) or getattr(node.target, "__name__", "") == "getitem":
                aliases.add(node)
        elif node.op == "call_method":
            name = node.target
            if name.endswith("_") and not name.endswith("__") and hasattr(torch.Tensor, name[:-1]):
                node.target = name[:-1]
            elif name in view_methods:
                aliases.add(node)
        elif node.op == "call_module" and owner is not None:
            sub = owner.get_submodule(node.target)
            if getattr(sub, "inplace", False):
                sub.inplace = False
    module.recompile()
    return module


def prune_graph(graph: fx.GraphModule) -> fx.GraphModule:
    """Dead-code elimination from the outputs (only sound for side-effect-free graphs)."""
    alive = set()
    stack = [n for n in graph.graph.nodes if n.op == "output"]
    while stack:
        node = stack.pop()
        if node in alive:
            continue
        alive.add(node)
        stack.extend(node.all_input_nodes)
    for node in reversed(list(graph.graph.nodes)):
        if node not in alive and node.op not in ("placeholder", "output"):
            graph.graph.erase_node(node)
    graph.recompile()
    return graph


_PALETTE = ["#a6cee3", "#b2df8a", "#fb9a99", "#fdbf6f", "#cab2d6", "#ffff99", "#1f78b4", "#33a02c", "#e31a1c", "#ff7f00", "#6a3d9a", "#b15928"]


def partition_to_dot(parts: List[List[fx.Node]], out: Optional[TextIO] = None) -> str:
    """DOT text with one coloured cluster per part."""
    lines = ["digraph partition {", "  node [style=filled, shape=box, fontsize=10];"]
    home = {}
    for i, part in enumerate(parts):
        lines.append(f"  subgraph cluster_{i} {{")
        lines.append(f'    label="part {i}"; color="{_PALETTE[i % len(_PALETTE)]}";')
        for nd in part:
            home[nd] = i
            lines.append(f'    "{nd.name}" [fillcolor="{_PALETTE[i % len(_PALETTE)]}"];')
        lines.append("  }")
    for part in parts:
        for nd in part:
            for dep in nd.all_input_nodes:
                if dep in home:
                    style = "" if home[dep] == home[nd] else ' [color=red, penwidth=2]'
                    lines.append(f'  "{dep.name}" -> "{nd.name}"{style};')
    lines.append("}")
    text = "\n".join(lines)
    if out is not None:
        out.write(text)
    return text


def export_partition_to_image(parts: List[List[fx.Node]], filename: str, format: str = "png") -> str:
    """Render with Graphviz ``dot`` when installed; otherwise write the DOT text next to
    the requested file and return that path."""
    text = partition_to_dot(parts)
    exe = shutil.which("dot")
    if exe is None:
        path = filename + ".dot"
        with open(path, "w") as f:
            f.write(text)
        print(f"graphviz 'dot' not found; wrote {path}", file=sys.stderr)
        return path
    subprocess.run([exe, f"-T{format}", "-o", filename], input=text.encode(), check=True)
    return filename
