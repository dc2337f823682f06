"""``metis`` partitioner: ``gpmetis`` when the program is installed, else the in-tree
minimum-volume partitioner (``elf_b200/partitioners/dag.py``).

The external path follows the reference's recipe (``elf/partitioners/metis.py``): node times
and edge bytes are rescaled to integers in [1, 100] (edges that are not tensors get a
prohibitive weight), the graph is written in METIS format ``110`` (node weights and edge
weights, one constraint) and ``gpmetis`` is run with the volume objective and contiguous,
minimally connected parts.
"""

from __future__ import annotations

import logging
import os
import shutil
import subprocess
import tempfile
from typing import Dict, List

import torch.fx as fx

from .custom import _nodes_of
from .dag import split_graph_min_volume
from .profile import DONT_CUT_HERE

logger = logging.getLogger("partition")

__all__ = ["split_graph_metis", "write_metis", "read_parts", "rescale"]


def rescale(values: List[float], lo: int = 1, hi: int = 100) -> List[int]:
    finite = [v for v in values if v < DONT_CUT_HERE]
    top = max(finite, default=0.0)
    out = []
    for v in values:
        if v >= DONT_CUT_HERE:
            out.append(DONT_CUT_HERE)
        elif top <= 0:
            out.append(lo)
        else:
            out.append(max(lo, min(hi, int(round(lo + (hi - lo) * v / top)))))
    return out


def write_metis(path: str, nodes: List[fx.Node], times: Dict[str, float], memories: Dict[str, float]) -> None:
    index = {nd: i + 1 for i, nd in enumerate(nodes)}
    w_node = rescale([float(times.get(nd.name, 0)) for nd in nodes])
    w_out = dict(zip(nodes, rescale([float(memories.get(nd.name, 0)) for nd in nodes])))
    adj: Dict[fx.Node, Dict[fx.Node, int]] = {nd: {} for nd in nodes}
    for nd in nodes:
        for dep in nd.all_input_nodes:
            if dep in index and dep is not nd:
                adj[nd][dep] = w_out[dep]
                adj[dep][nd] = w_out[dep]
    n_edges = sum(len(a) for a in adj.values()) // 2
    with open(path, "w") as f:
        f.write(f"{len(nodes)} {n_edges} 110 1\n")
        for nd, w in zip(nodes, w_node):
            f.write(" ".join([str(w)] + [f"{index[o]} {ew}" for o, ew in adj[nd].items()]) + "\n")


def read_parts(path: str, nodes: List[fx.Node], n: int) -> List[List[fx.Node]]:
    with open(path) as f:
        owner = [int(line) for line in f.read().split()]
    parts: List[List[fx.Node]] = [[] for _ in range(n)]
    for nd, p in zip(nodes, owner):
        parts[p].append(nd)
    return parts


def split_graph_metis(graph, times, memories, n: int) -> List[List[fx.Node]]:
    exe = shutil.which("gpmetis")
    if exe is None:
        logger.info("gpmetis not found: using the in-tree minimum-volume partitioner")
        return split_graph_min_volume(graph, times, memories, n, ratio=1.1)
    nodes = _nodes_of(graph)
    with tempfile.TemporaryDirectory() as tmp:
        path = os.path.join(tmp, "graph.metis")
        write_metis(path, nodes, times, memories)
        subprocess.run([exe, path, str(n), "-objtype=vol", "-contig", "-minconn", "-ufactor=100", "-ncuts=200", "-niter=200"], check=True, capture_output=True)
        return read_parts(f"{path}.part.{n}", nodes, n)
