"""From a list-of-node-lists to runnable stage modules.

``partition(model, n, sample, partitioner, tracer)`` traces, profiles and cuts a model and
returns a ``PartitionResult`` (signatures, estimated times/transfers, balance and transfer
scores, ``create_blocks()``, ``validate()``, ``to_image()``), as in the reference
(``elf/partitioners/partition.py``).  Two things are done differently:

* ``get_attr`` nodes (how ``torch.export`` graphs reference parameters) are moved into the
  part of their first user before inputs/outputs are derived, so weights never become
  stage inputs that would travel over p2p every micro-batch;
* the ``metis``/``dagP`` keys run an in-tree partitioner when their external program is
  missing instead of degrading to ``naive``.
"""

from __future__ import annotations

import logging
from typing import Dict, List, Optional, Set

import torch.fx as fx

from ..registry import PARTITIONERS, resolve
from .profile import profile_operations
from .signature import Signature
from .tracing import trace
from .utils import export_partition_to_image, remove_inplace_leaves

logger = logging.getLogger("partition")

__all__ = [
    "PartitionResult",
    "partition",
    "split",
    "check_partition",
    "create_subgraph",
    "get_inputs_outputs",
    "get_sources_targets",
    "pin_get_attrs",
]


def _scalar(x) -> float:
    return float(x.item()) if hasattr(x, "item") else float(x)


class PartitionResult:
    def __init__(self, graph_module: fx.GraphModule, parts: List[List[fx.Node]], inputs: Dict[int, List[str]], outputs: Dict[int, List[str]], times: Dict[str, float], memories: Dict[str, float]):
        self.graph_module = graph_module
        self.parts = parts
        self.inputs = inputs
        self.outputs = outputs
        self.times = times
        self.memories = memories
        self._signatures: Optional[List[Signature]] = None

    @property
    def n(self) -> int:
        return len(self.parts)

    @property
    def signatures(self) -> List[Signature]:
        if self._signatures is None:
            sources, targets = get_sources_targets(self.inputs, self.outputs)
            self._signatures = [Signature(self.inputs[i], self.outputs[i], sources[i], targets[i]) for i in range(self.n)]
        return self._signatures

    @property
    def estimated_times(self) -> List[float]:
        """Seconds per part (sum of the profiled node times)."""
        return [_scalar(sum(self.times.get(nd.name, 0) for nd in part)) for part in self.parts]

    @property
    def estimated_memory_transfers(self) -> List[float]:
        """MB leaving each part."""
        return [sum(self.memories.get(o, 0) for o in self.outputs[i]) / 2**20 for i in range(self.n)]

    @property
    def balance_score(self) -> float:
        """``max_p T_p / mean_p T_p`` — 1 is perfect."""
        t = self.estimated_times
        mean = sum(t) / self.n
        return max(t) / mean if mean > 0 else 1.0

    @property
    def transfer_score(self) -> float:
        """MB crossing stage boundaries (the last part sends to nobody)."""
        return sum(self.estimated_memory_transfers[:-1])

    def create_blocks(self) -> List[fx.GraphModule]:
        blocks = []
        for i, part in enumerate(self.parts):
            sub = create_subgraph(self.graph_module, part, self.inputs[i], self.outputs[i])
            remove_inplace_leaves(sub)
            blocks.append(sub)
        return blocks

    def validate(self) -> None:
        check_partition(self.graph_module.graph, self.parts, self.inputs, self.outputs)

    def to_image(self, filename: str, format: str = "png") -> str:
        return export_partition_to_image(self.parts, filename, format)

    def __repr__(self) -> str:
        return f"PartitionResult(n={self.n}, estimated_times=[{', '.join(f'{t:.3f}s' for t in self.estimated_times)}])"


def check_partition(graph, parts, inputs, outputs) -> None:
    original = [nd.target for nd in graph.nodes if nd.op == "placeholder"]
    if sorted(original) != sorted(inputs[0]):
        raise Exception(f"Inputs of the first part do not match original inputs: {original} != {inputs[0]}")
    available: Set[str] = set(outputs[0])
    for i in range(1, len(parts)):
        if len(parts[i]) == 0:
            raise Exception(f"Part {i} is empty")
        for name in inputs[i]:
            if name not in available:
                raise Exception(f"Input {name} of part {i} is not an output of any previous part")
        available.update(outputs[i])


def create_subgraph(graph_module: fx.GraphModule, nodes: List[fx.Node], inputs: List[str], outputs: List[str]) -> fx.GraphModule:
    """``fx.GraphModule`` computing ``outputs`` (returned as a tuple) from ``inputs``.  The
    sub-module shares the original module's parameters and keeps their qualified names."""
    sub = fx.Graph()
    env: Dict[str, fx.Node] = {}
    for name in inputs:
        node = sub.placeholder(name)
        env[name] = node
        env[node.name] = node  # fx may rename (a placeholder called `input` becomes `input_1`)
    for nd in nodes:
        env[nd.name] = sub.node_copy(nd, lambda a: env[a.name])
    sub.output(tuple(env[o] for o in outputs))
    sub.lint()
    return fx.GraphModule(graph_module, sub)


def pin_get_attrs(parts: List[List[fx.Node]]) -> List[List[fx.Node]]:
    """Move every ``get_attr`` node into the part of its earliest user (duplicating it for
    users in later parts is unnecessary: the value then flows as an ordinary tensor)."""
    home = {nd: i for i, part in enumerate(parts) for nd in part}
    moved: Dict[fx.Node, int] = {}
    for i, part in enumerate(parts):
        for nd in part:
            if nd.op != "get_attr":
                continue
            users = [home[u] for u in nd.users if u in home]
            if users and min(users) != i:
                moved[nd] = min(users)
    if not moved:
        return parts
    out = [[nd for nd in part if nd not in moved] for part in parts]
    for nd, dst in moved.items():
        out[dst].insert(0, nd)
    return out


def pin_placeholders(parts: List[List[fx.Node]]) -> List[List[fx.Node]]:
    """All model inputs enter through the first part (the only stage the runtime feeds);
    later parts that use one receive it as a pass-through output of that part."""
    strays = [nd for part in parts[1:] for nd in part if nd.op == "placeholder"]
    if not strays:
        return parts
    out = [[nd for nd in part if nd not in strays] for part in parts]
    out[0] = strays + out[0]
    return out


def _part_io(parts: List[List[fx.Node]]):
    n = len(parts)
    home = {nd: i for i, part in enumerate(parts) for nd in part}
    inputs: Dict[int, List[str]] = {i: [] for i in range(n)}
    outputs: Dict[int, List[str]] = {i: [] for i in range(n)}
    deps: Dict[int, Set[int]] = {i: set() for i in range(n)}

    def add_final_outputs(i, arg):
        if isinstance(arg, (list, tuple)):
            for a in arg:
                add_final_outputs(i, a)
        elif isinstance(arg, dict):
            for a in arg.values():
                add_final_outputs(i, a)
        elif isinstance(arg, fx.Node):
            src = home.get(arg, i)
            if arg.name not in outputs[src]:
                outputs[src].append(arg.name)

    for i, part in enumerate(parts):
        for nd in part:
            if nd.op == "placeholder":
                if nd.target not in inputs[i]:
                    inputs[i].append(nd.target)
                continue
            if nd.op == "output":
                for arg in nd.args:
                    add_final_outputs(i, arg)
                continue
            for dep in nd.all_input_nodes:
                src = home.get(dep)
                if src == i:
                    if dep.op == "placeholder" and dep.target not in inputs[i]:
                        inputs[i].append(dep.target)
                    continue
                # a value made (or, for a model input, received) by another part
                name = dep.target if dep.op == "placeholder" else dep.name
                if name not in inputs[i]:
                    inputs[i].append(name)
                if src is not None:
                    if name not in outputs[src]:
                        outputs[src].append(name)
                    deps[i].add(src)
    return inputs, outputs, deps


def _topo_order(deps: Dict[int, Set[int]]) -> List[int]:
    n = len(deps)
    remaining = {i: set(d) for i, d in deps.items()}
    order: List[int] = []
    ready = sorted(i for i in range(n) if not remaining[i])
    while ready:
        cur = ready.pop(0)
        order.append(cur)
        for i in range(n):
            if cur in remaining[i]:
                remaining[i].discard(cur)
                if not remaining[i] and i not in order and i not in ready:
                    ready.append(i)
        ready.sort()
    if len(order) != n:
        raise Exception("Cycle detected in partition dependencies")
    return order


def get_inputs_outputs(parts: List[List[fx.Node]]):
    """Inputs/outputs per part (sorted names), parts in dependency order, without their
    placeholder/output nodes.  A final output produced by an earlier part than the one
    holding the graph's ``output`` node is exported by its producer."""
    parts = pin_placeholders(pin_get_attrs(parts))
    inputs, outputs, deps = _part_io(parts)
    order = _topo_order(deps)
    parts = [parts[i] for i in order]
    inputs = {new: sorted(inputs[old]) for new, old in enumerate(order)}
    outputs = {new: sorted(outputs[old]) for new, old in enumerate(order)}
    parts = [[nd for nd in part if nd.op not in ("placeholder", "output")] for part in parts]
    return parts, inputs, outputs


def get_sources_targets(inputs: Dict[int, List[str]], outputs: Dict[int, List[str]]):
    """``sources[i][k]``: part producing input ``k`` of part ``i`` (``None`` = model input);
    ``targets[i][k]``: parts consuming output ``k`` (``[None]`` = model output)."""
    n = len(inputs)
    producer: Dict[str, int] = {}
    for i in range(n):
        for o in outputs[i]:
            producer.setdefault(o, i)
    sources = [[producer[name] if name in producer and producer[name] < i else None for name in inputs[i]] for i in range(n)]
    targets = []
    for i in range(n):
        row = []
        for o in outputs[i]:
            users = [j for j in range(i + 1, n) if o in inputs[j]]
            row.append(users or [None])
        targets.append(row)
    return sources, targets


def split(graph_module: fx.GraphModule, times, memories, n: int, partitioner="constrained") -> PartitionResult:
    fn = resolve(partitioner, PARTITIONERS)
    raw = fn(graph_module, times, memories, n)
    assert len(raw) == n, f"Expected {n} parts, got {len(raw)}"
    parts, inputs, outputs = get_inputs_outputs(raw)
    result = PartitionResult(graph_module, parts, inputs, outputs, times, memories)
    result.validate()
    return result


def partition(model, n: int, sample, partitioner="constrained", tracer="default") -> PartitionResult:
    """Trace, profile and cut ``model`` into ``n`` parts."""
    model.train()
    gm = trace(model, sample, tracer)
    logger.info("Extracted graph has %d nodes", len(gm.graph.nodes))
    times, memories = profile_operations(gm, sample)
    result = split(gm, times, memories, n, partitioner)
    logger.info("Estimated times: %s", ["%.3fs" % t for t in result.estimated_times])
    logger.info("Estimated memory transfers: %s", ["%.1fMB" % m for m in result.estimated_memory_transfers])
    return result
