"""``dagP`` partitioner: the external acyclic partitioner ``rMLGP`` when installed
(reference ``elf/partitioners/dagP.py:13-98``: DOT input, ``--ratio 1.3``, 100 runs), else the
in-tree acyclic minimum-volume partitioner with the same balance ratio."""

from __future__ import annotations

import logging
import os
import shutil
import subprocess
import tempfile
from typing import List

import torch.fx as fx

from .custom import _nodes_of
from .dag import split_graph_min_volume
from .metis import read_parts, rescale

logger = logging.getLogger("partition")

__all__ = ["split_graph_dagP", "write_dot"]


def write_dot(path: str, nodes: List[fx.Node], times, memories) -> None:
    index = {nd: i for i, nd in enumerate(nodes)}
    w_node = rescale([float(times.get(nd.name, 0)) for nd in nodes])
    w_out = dict(zip(nodes, rescale([float(memories.get(nd.name, 0)) for nd in nodes])))
    with open(path, "w") as f:
        f.write("digraph G {\n")
        for nd, w in zip(nodes, w_node):
            f.write(f'{index[nd]} [weight="{w}"];\n')
        for nd in nodes:
            for dep in nd.all_input_nodes:
                if dep in index:
                    f.write(f'{index[dep]}->{index[nd]} [weight="{w_out[dep]}"];\n')
        f.write("}\n")


def split_graph_dagP(graph, times, memories, n: int) -> List[List[fx.Node]]:
    exe = shutil.which("rMLGP")
    if exe is None:
        logger.info("rMLGP not found: using the in-tree acyclic minimum-volume partitioner")
        return split_graph_min_volume(graph, times, memories, n, ratio=1.3)
    nodes = _nodes_of(graph)
    with tempfile.TemporaryDirectory() as tmp:
        path = os.path.join(tmp, "graph.dot")
        write_dot(path, nodes, times, memories)
        subprocess.run([exe, path, str(n), "--obj", "1", "--write_parts", "1", "--print", "0", "--ratio", "1.3", "--runs", "100"], check=True, capture_output=True)
        produced = [p for p in os.listdir(tmp) if ".part" in p or "partsfile" in p]
        if not produced:
            raise RuntimeError("rMLGP wrote no parts file")
        return read_parts(os.path.join(tmp, sorted(produced)[0]), nodes, n)
