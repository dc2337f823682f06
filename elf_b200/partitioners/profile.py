"""Per-node forward cost of a traced model: seconds and output bytes.

An ``fx.Interpreter`` re-runs every node ``niter`` times and keeps the median.  Unlike the
reference profiler (``elf/partitioners/profile.py:14-164``), which shuttles each node's
arguments and module between CPU and GPU around every measurement, the graph stays on
one device for the whole run and CUDA timings are read from events after a single
synchronisation per node.  Nodes whose output is not a tensor get the sentinel cost
``DONT_CUT_HERE`` as "memory" so no partitioner cuts an edge that cannot be sent.
"""

from __future__ import annotations

import copy
import statistics
import time
from typing import Dict, Tuple

import torch
import torch.fx as fx

from ..zb_utils import LayerDW

__all__ = ["Profiler", "profile_operations", "get_memory", "DONT_CUT_HERE"]

DONT_CUT_HERE = 2 << 24


def get_memory(x) -> float:
    """Bytes of a tensor (or of all tensors of a tuple/list of tensors); ``DONT_CUT_HERE`` otherwise."""
    if isinstance(x, torch.Tensor):
        return x.numel() * x.element_size()
    if isinstance(x, (tuple, list)) and x and all(isinstance(t, torch.Tensor) for t in x):
        return DONT_CUT_HERE  # a tuple cannot travel as one message
    return DONT_CUT_HERE


class Profiler(fx.Interpreter):
    def __init__(self, niter: int, module: fx.GraphModule, device=None):
        super().__init__(module, garbage_collect_values=True)
        self.niter = max(1, niter)
        self.times: Dict[str, float] = {}
        self.memories: Dict[str, float] = {}
        self.device = torch.device(device) if device is not None else None
        self._cuda = self.device is not None and self.device.type == "cuda"

    def run_node(self, node):
        if node.op == "call_module":
            mod = self.fetch_attr(node.target)
            if isinstance(mod, LayerDW):
                mod.last_input = None
        if node.op in ("placeholder", "output", "get_attr"):
            result = super().run_node(node)
            self.times[node.name] = 0.0
            self.memories[node.name] = get_memory(result) if node.op != "output" else 0
            return result
        samples = []
        result = None
        if self._cuda:
            events = []
            for _ in range(self.niter):
                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a.record()
                result = super().run_node(node)
                b.record()
                events.append((a, b))
            torch.cuda.synchronize(self.device)
            samples = [a.elapsed_time(b) / 1e3 for a, b in events]
        else:
            for _ in range(self.niter):
                t0 = time.perf_counter()
                result = super().run_node(node)
                samples.append(time.perf_counter() - t0)
        self.times[node.name] = statistics.median(samples)
        self.memories[node.name] = get_memory(result)
        if node.op == "call_module":
            mod = self.fetch_attr(node.target)
            if isinstance(mod, LayerDW):
                mod.last_input = None
        return result


def _first_device(module: torch.nn.Module):
    for t in list(module.parameters()) + list(module.buffers()):
        if not t.is_meta:
            return t.device
    return torch.device("cpu")


def profile_operations(graph_module: fx.GraphModule, input_sample, niter: int = 10) -> Tuple[Dict[str, float], Dict[str, float]]:
    """``({node name: seconds}, {node name: output bytes})`` of one forward on ``input_sample``
    (tensor, list/tuple of tensors, or dict in placeholder order).  Buffers are restored
    afterwards (BatchNorm statistics and the like must not drift)."""
    if isinstance(input_sample, torch.Tensor):
        inputs = [input_sample]
    elif isinstance(input_sample, dict):
        inputs = list(input_sample.values())
    else:
        inputs = list(input_sample)
    n_placeholders = sum(1 for n in graph_module.graph.nodes if n.op == "placeholder")
    assert n_placeholders == len(inputs), f"Expected {n_placeholders} inputs, got {len(inputs)}"

    device = _first_device(graph_module)
    saved = {name: buf.detach().clone() for name, buf in graph_module.named_buffers()}
    inputs = [t.to(device) if isinstance(t, torch.Tensor) else t for t in inputs]
    prof = Profiler(niter, graph_module, device)
    with torch.no_grad():
        prof.run(*copy.copy(inputs))
    for name, buf in graph_module.named_buffers():
        buf.data.copy_(saved[name])
    for node in graph_module.graph.nodes:
        prof.times.setdefault(node.name, 0.0)
        prof.memories.setdefault(node.name, 0)
    return prof.times, prof.memories
