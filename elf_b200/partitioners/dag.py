"""In-tree acyclic k-way partitioner with a communication-volume objective.

The reference delegates its ``metis`` and ``dagP`` partitioners to the external programs
``gpmetis`` (``elf/partitioners/metis.py:230-254``: volume objective, contiguous parts,
``ufactor=100``) and ``rMLGP`` (``elf/partitioners/dagP.py:75-92``: acyclic parts,
``--ratio 1.3``) and silently degrades to the naive splitter when they are not installed
(``elf/partitioners/partition.py:130-147``).  This module serves both registry keys when
the binaries are absent.

Parts are contiguous ranges of a topological order, which makes them acyclic by
construction.  With ``cost(i)`` = bytes crossing a cut before node ``i`` and part loads
bounded by ``ratio · total / n``, the cut set of minimum total volume is found by dynamic
programming with a sliding-window minimum (``O(n · N)``); if the balance bound admits no
solution it is relaxed geometrically.
"""

from __future__ import annotations

import logging
from collections import deque
from typing import Dict, List

import torch.fx as fx

from .custom import _nodes_of, cut_bytes, cut_widths, split_graph

logger = logging.getLogger("partition")

__all__ = ["split_graph_min_volume"]

_INF = float("inf")


def _native_solver():
    """The C++ implementation of ``_solve`` (``csrc/host_runtime.cpp``) when the extension is built."""
    try:
        from ..ops import _ext

        if _ext.available():
            return getattr(_ext.get(), "min_volume_cuts", None)
    except Exception:  # the extension is optional for the front-end
        pass
    return None


def _solve(prefix: List[float], cost: List[float], allowed: List[bool], n_parts: int, cap: float, native: bool = True):
    solver = _native_solver() if native else None
    if solver is not None and cap != _INF:
        cuts = solver(list(map(float, prefix)), list(map(float, cost)), list(map(bool, allowed)), int(n_parts), float(cap))
        return [int(c) for c in cuts] if len(cuts) == n_parts - 1 and (n_parts > 1) else None
    n = len(prefix) - 1
    # best[k][i]: cheapest way to close k parts with the k-th ending right before node i
    best = [[_INF] * (n + 1) for _ in range(n_parts + 1)]
    back = [[-1] * (n + 1) for _ in range(n_parts + 1)]
    best[0][0] = 0.0
    for k in range(1, n_parts + 1):
        window: deque = deque()  # candidate starts j, increasing best[k-1][j]
        j_next = 0
        for i in range(1, n + 1):
            while j_next < i:
                if best[k - 1][j_next] < _INF:
                    while window and best[k - 1][window[-1]] >= best[k - 1][j_next]:
                        window.pop()
                    window.append(j_next)
                j_next += 1
            while window and prefix[i] - prefix[window[0]] > cap:
                window.popleft()
            if not window:
                continue
            last = k == n_parts
            if last and i != n:
                continue
            if not last and not allowed[i]:
                continue
            j = window[0]
            best[k][i] = best[k - 1][j] + (0.0 if last else cost[i])
            back[k][i] = j
    if best[n_parts][n] == _INF:
        return None
    cuts, i = [], n
    for k in range(n_parts, 0, -1):
        i = back[k][i]
        cuts.append(i)
    return sorted(cuts)[1:]  # drop the leading 0


def split_graph_min_volume(graph, times: Dict[str, float], memories: Dict[str, float], n: int, ratio: float = 1.3) -> List[List[fx.Node]]:
    nodes = _nodes_of(graph)
    if n == 1:
        return [nodes]
    prefix = [0.0]
    for nd in nodes:
        prefix.append(prefix[-1] + float(times.get(nd.name, 0)))
    total = prefix[-1]
    cost = cut_bytes(nodes, memories)
    width, ok = cut_widths(nodes, memories)
    first_real = next((i for i, nd in enumerate(nodes) if nd.op not in ("placeholder", "get_attr")), 0)
    last_real = max((i for i, nd in enumerate(nodes) if nd.op != "output"), default=len(nodes) - 1)
    allowed = [ok[i] and width[i] > 0 and first_real < i <= last_real for i in range(len(nodes) + 1)]
    r = ratio
    for _ in range(12):
        cuts = _solve(prefix, cost, allowed, n, r * total / n if total > 0 else _INF)
        if cuts is not None and len(cuts) == n - 1:
            bounds = [0] + cuts + [len(nodes)]
            return [nodes[bounds[k] : bounds[k + 1]] for k in range(n)]
        r *= 1.5
    logger.warning("min-volume partitioner found no balanced cut set; falling back to naive")
    return split_graph(graph, times, memories, n)
