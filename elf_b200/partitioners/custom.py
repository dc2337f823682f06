"""Built-in partitioners over the topological node order of an fx graph.

``naive``        greedy prefix cuts whenever the running time passes ``k·total/n``
                 (reference ``elf/partitioners/custom.py:10-45``).
``constrained``  (default) cuts are allowed only where at most ``max_cuts`` live tensors
                 cross; among those positions the cut set minimising the heaviest part is
                 found *exactly* (bottleneck search over candidate positions) for
                 ``max_cuts`` = 1..10 and the best ``max/avg + 0.1·(max_cuts − 1)`` wins.
                 Same objective and penalty as the reference's reverse sweep with a growing
                 imbalance margin (``:48-141``), without its heuristics.
"""

from __future__ import annotations

import bisect
import logging
from typing import Dict, List, Optional, Sequence

import torch.fx as fx

from .profile import DONT_CUT_HERE

logger = logging.getLogger("partition")

__all__ = ["split_graph", "split_graph_constrained", "cut_widths", "cut_bytes", "_evaluate_partition_balance"]


def _nodes_of(graph) -> List[fx.Node]:
    g = graph.graph if hasattr(graph, "graph") else graph
    return list(g.nodes)


def _evaluate_partition_balance(parts, times) -> float:
    if any(len(p) == 0 for p in parts):
        return float("inf")
    loads = [sum(times.get(n.name, 0) for n in part) for part in parts]
    avg = sum(loads) / len(loads)
    return max(loads) / avg if avg > 0 else 1.0


def split_graph(graph, times: Dict[str, float], memories: Dict[str, float], n: int) -> List[List[fx.Node]]:
    nodes = _nodes_of(graph)
    total = sum(times.get(nd.name, 0) for nd in nodes)
    parts: List[List[fx.Node]] = [[] for _ in range(n)]
    acc, k = 0.0, 0
    for i, nd in enumerate(nodes):
        remaining_nodes = len(nodes) - i
        # leave at least one node for every part still to be opened
        if k < n - 1 and parts[k] and (acc >= (k + 1) * total / n or remaining_nodes <= n - 1 - k):
            k += 1
        parts[k].append(nd)
        acc += times.get(nd.name, 0)
    return parts


def _live_ranges(nodes: Sequence[fx.Node]):
    pos = {nd: i for i, nd in enumerate(nodes)}
    last_use = [i for i in range(len(nodes))]
    for nd in nodes:
        for dep in nd.all_input_nodes:
            if dep in pos:
                last_use[pos[dep]] = max(last_use[pos[dep]], pos[nd])
    return pos, last_use


def cut_widths(nodes: Sequence[fx.Node], memories: Optional[Dict[str, float]] = None):
    """``width[i]`` = number of values defined before position ``i`` and used at or after it
    (what a cut *before* node ``i`` would have to transfer); ``ok[i]`` is False when one of
    them is not a tensor.  Parameters fetched by ``get_attr`` never count: they are moved
    next to their user when sub-graphs are built."""
    n = len(nodes)
    _, last_use = _live_ranges(nodes)
    delta = [0] * (n + 2)
    bad = [0] * (n + 2)
    for i, nd in enumerate(nodes):
        if nd.op in ("output", "get_attr") or last_use[i] <= i:
            continue
        delta[i + 1] += 1
        delta[last_use[i] + 1] -= 1
        if memories is not None and memories.get(nd.name, 0) >= DONT_CUT_HERE:
            bad[i + 1] += 1
            bad[last_use[i] + 1] -= 1
    width, ok = [0] * (n + 1), [True] * (n + 1)
    w = b = 0
    for i in range(n + 1):
        w += delta[i]
        b += bad[i]
        width[i], ok[i] = w, b == 0
    return width, ok


def cut_bytes(nodes: Sequence[fx.Node], memories: Dict[str, float]) -> List[float]:
    """Bytes crossing a cut before each position (sentinel-sized for non-tensors)."""
    n = len(nodes)
    _, last_use = _live_ranges(nodes)
    delta = [0.0] * (n + 2)
    for i, nd in enumerate(nodes):
        if nd.op in ("output", "get_attr") or last_use[i] <= i:
            continue
        m = float(memories.get(nd.name, 0))
        delta[i + 1] += m
        delta[last_use[i] + 1] -= m
    out, acc = [0.0] * (n + 1), 0.0
    for i in range(n + 1):
        acc += delta[i]
        out[i] = acc
    return out


def _bottleneck_cuts(prefix: List[float], candidates: List[int], n_parts: int, n_nodes: int) -> Optional[List[int]]:
    """Choose ``n_parts − 1`` cut positions among ``candidates`` (sorted) minimising the
    largest segment sum; ``None`` if there are too few candidates."""
    if len(candidates) < n_parts - 1:
        return None
    total = prefix[n_nodes]

    def greedy(limit: float) -> Optional[List[int]]:
        cuts, start = [], 0
        for part in range(n_parts - 1):
            # furthest candidate whose segment [start, c) stays within the limit, leaving
            # enough candidates for the parts still to be closed
            hi = bisect.bisect_right(candidates, start)
            best = None
            max_idx = len(candidates) - (n_parts - 1 - part - 1) - 1
            for idx in range(hi, max_idx + 1):
                c = candidates[idx]
                if prefix[c] - prefix[start] <= limit + 1e-15:
                    best = c
                else:
                    break
            if best is None:
                return None
            cuts.append(best)
            start = best
        return cuts if total - prefix[start] <= limit + 1e-15 else None

    lo, hi = total / n_parts, total
    best = greedy(hi)
    if best is None:
        return None
    for _ in range(50):
        mid = 0.5 * (lo + hi)
        trial = greedy(mid)
        if trial is None:
            lo = mid
        else:
            hi, best = mid, trial
        if hi - lo <= 1e-9 * max(total, 1e-30):
            break
    return best


def split_graph_constrained(graph, times: Dict[str, float], memories: Dict[str, float], n: int, cut_penalty: float = 0.1, max_cuts_limit: int = 10) -> List[List[fx.Node]]:
    nodes = _nodes_of(graph)
    if n == 1:
        return [nodes]
    width, ok = cut_widths(nodes, memories)
    prefix = [0.0]
    for nd in nodes:
        prefix.append(prefix[-1] + float(times.get(nd.name, 0)))
    # a cut must leave at least one real node on each side
    first_real = next((i for i, nd in enumerate(nodes) if nd.op not in ("placeholder", "get_attr")), 0)
    last_real = max((i for i, nd in enumerate(nodes) if nd.op != "output"), default=len(nodes) - 1)
    best_parts, best_score = None, float("inf")
    for max_cuts in range(1, max_cuts_limit + 1):
        cands = [i for i in range(first_real + 1, last_real + 1) if ok[i] and 0 < width[i] <= max_cuts]
        cuts = _bottleneck_cuts(prefix, cands, n, len(nodes))
        if cuts is None:
            continue
        bounds = [0] + cuts + [len(nodes)]
        parts = [nodes[bounds[k] : bounds[k + 1]] for k in range(n)]
        score = _evaluate_partition_balance(parts, times) + (max_cuts - 1) * cut_penalty
        if score < best_score - 1e-12:
            best_score, best_parts = score, parts
            logger.debug("constrained: score %.4f with at most %d tensors per cut", score, max_cuts)
    if best_parts is None:
        logger.warning("constrained partitioner found no admissible cut set; falling back to naive")
        return split_graph(graph, times, memories, n)
    return best_parts
