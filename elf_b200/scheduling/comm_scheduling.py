"""Communication insertion and deadlock-free ordering of p2p operations.

``add_comms`` attaches RECV/SEND ops to every forward and backward-inputs op according to
the stage signatures and appends one ALL_REDUCE_PARAM_GRADS per stage
(reference ``elf/scheduling/comm_scheduling.py:557-598``).  The three comm schedulers
(``topo``, ``simulation``, ``pipelined``; reference ``:172-450``) then produce one global
order whose per-rank projection is what each rank executes.

All three run on one dependency model (``_Plan``) built in a single pass with hash lookups:

* ``F(s, mb)`` waits for its RECV_FORWARDs, ``SEND_FORWARD`` for its ``F``;
  same for ``B`` with RECV/SEND_BACKWARD; a last-stage RECV_BACKWARD waits for LOSS_BACKWARD;
* compute, loss, recompute, all-reduce and prefetch ops keep their per-rank program order;
* a send and its recv form a *pair*: whoever consumes the recv also waits for the send
  to be issued, and a comm op is *ready* when both ends have no other unmet dependency.

Each scheduler is a different emission policy over that model, so its cost is linear in
the number of ops per round instead of the reference's quadratic scans.
"""

from __future__ import annotations

import heapq
from collections import defaultdict
from typing import Dict, Iterable, List, Optional, Set, Tuple

from .scheduling import (
    Operation,
    OperationType,
    comm_types,
    compute_types,
    get_peer,
    matching,
    recv_types,
    send_types,
)
from ..partitioners.signature import Signature

__all__ = [
    "DirectedGraph",
    "add_comms",
    "schedule_to_graph",
    "topological_sort",
    "smart_topological_sort",
    "pipelined_topological_sort",
]

T = OperationType


class DirectedGraph:
    """Directed graph on nodes ``0..n-1`` with ordered adjacency sets."""

    def __init__(self, num_nodes: int):
        if num_nodes <= 0:
            raise ValueError("Number of nodes must be positive")
        self.num_nodes = num_nodes
        self._succ: List[Dict[int, None]] = [dict() for _ in range(num_nodes)]
        self._pred: List[Dict[int, None]] = [dict() for _ in range(num_nodes)]

    def _check(self, *nodes: int) -> None:
        for v in nodes:
            if not 0 <= v < self.num_nodes:
                raise ValueError("Node indices must be within valid range")

    def add_edge(self, source: int, target: int) -> None:
        self._check(source, target)
        if source == target:
            raise ValueError("Self-loops are not allowed")
        self._succ[source][target] = None
        self._pred[target][source] = None

    def remove_edge(self, source: int, target: int) -> None:
        self._succ[source].pop(target, None)
        self._pred[target].pop(source, None)

    def has_edge(self, source: int, target: int) -> bool:
        return target in self._succ[source]

    def has_unidirectional_edge(self, a: int, b: int) -> bool:
        return self.has_edge(a, b) and not self.has_edge(b, a)

    def has_bidirectional_edge(self, a: int, b: int) -> bool:
        return self.has_edge(a, b) and self.has_edge(b, a)

    def get_successors(self, node: int) -> List[int]:
        return list(self._succ[node])

    def get_predecessors(self, node: int) -> List[int]:
        return list(self._pred[node])

    def get_in_degree(self, node: int) -> int:
        return len(self._pred[node])

    def get_out_degree(self, node: int) -> int:
        return len(self._succ[node])

    @property
    def edges(self) -> Set[Tuple[int, int]]:
        return {(u, v) for u in range(self.num_nodes) for v in self._succ[u]}

    def has_cycle(self) -> bool:
        """True if a cycle longer than 2 exists (a ↔ b pairs are not cycles here)."""
        WHITE, GREY, BLACK = 0, 1, 2
        colour = [WHITE] * self.num_nodes
        for root in range(self.num_nodes):
            if colour[root] != WHITE:
                continue
            stack = [(root, -1, iter(self._succ[root]))]
            colour[root] = GREY
            while stack:
                node, parent, it = stack[-1]
                advanced = False
                for nxt in it:
                    if nxt == parent and self.has_edge(nxt, node):
                        continue  # 2-cycle with the node we came from
                    if colour[nxt] == GREY:
                        return True
                    if colour[nxt] == WHITE:
                        colour[nxt] = GREY
                        stack.append((nxt, node, iter(self._succ[nxt])))
                        advanced = True
                        break
                if not advanced:
                    colour[node] = BLACK
                    stack.pop()
        return False


# ---------------------------------------------------------------------------------------
# comm insertion
# ---------------------------------------------------------------------------------------

_ATTACHED = {
    T.FORWARD: (T.RECV_FORWARD, T.SEND_FORWARD),
    T.BACKWARD_INPUTS: (T.RECV_BACKWARD, T.SEND_BACKWARD),
}


def _ordered(peers: Iterable, reverse: bool) -> list:
    peers = list(peers)
    real = sorted((p for p in peers if p is not None), reverse=reverse)
    return real + [p for p in peers if p is None]


def add_comms(schedule: List[Operation], signatures: List[Signature]) -> List[Operation]:
    """Append, in place, the comm ops implied by ``signatures`` and the per-stage
    gradient all-reduce.  Returns ``schedule``.

    Forward data flows source → block → target, backward the other way round, so a
    forward recv names a *source* and a backward recv a *target*.  Peers are visited in
    descending order for "from the sources" lists and ascending for "to the targets"
    lists (the reference's order); ``None`` peers produce pseudo-comms."""
    present = {(op.op, op.block_id, op.mb_id) for op in schedule}
    extra: List[Operation] = []
    for op in schedule:
        pair = _ATTACHED.get(op.op)
        if pair is None:
            continue
        recv_t, send_t = pair
        sig = signatures[op.block_id]
        fwd = op.op is T.FORWARD
        if (recv_t, op.block_id, op.mb_id) not in present:
            present.add((recv_t, op.block_id, op.mb_id))
            peers = _ordered(sig.get_all_sources(), True) if fwd else _ordered(sig.get_all_targets(), False)
            extra += [Operation(op.block_id, op.mb_id, recv_t, op.rank, src=p) for p in peers]
        if (send_t, op.block_id, op.mb_id) not in present:
            present.add((send_t, op.block_id, op.mb_id))
            peers = _ordered(sig.get_all_targets(), False) if fwd else _ordered(sig.get_all_sources(), True)
            extra += [Operation(op.block_id, op.mb_id, send_t, op.rank, dst=p) for p in peers]
    schedule.extend(extra)
    kinds = {op.op for op in schedule}
    # a schedule without any backward (inference) produces no gradients: nothing to exchange
    if T.ALL_REDUCE_PARAM_GRADS not in kinds and kinds & {T.BACKWARD_INPUTS, T.BACKWARD_PARAMS}:
        for stage, rank in dict.fromkeys((op.block_id, op.rank) for op in schedule):
            schedule.append(Operation(stage, None, T.ALL_REDUCE_PARAM_GRADS, rank))
    return schedule


# ---------------------------------------------------------------------------------------
# dependency model
# ---------------------------------------------------------------------------------------

_ANCHORED = compute_types | {T.LOSS_FORWARD, T.LOSS_BACKWARD, T.ALL_REDUCE_PARAM_GRADS, T.PREFETCH_ACTIVATIONS}
_CHAIN = {
    T.FORWARD: T.RECV_FORWARD,
    T.SEND_FORWARD: T.FORWARD,
    T.BACKWARD_INPUTS: T.RECV_BACKWARD,
    T.SEND_BACKWARD: T.BACKWARD_INPUTS,
    T.RECV_BACKWARD: T.LOSS_BACKWARD,
}


class _Plan:
    def __init__(self, schedule: List[Operation]):
        self.ops = schedule
        n = len(schedule)
        self.users: List[List[int]] = [[] for _ in range(n)]
        self.unmet = [0] * n
        self.partner = [-1] * n
        self.emitted = [False] * n

        index: Dict[tuple, List[int]] = defaultdict(list)
        for i, op in enumerate(schedule):
            index[(op.block_id, op.mb_id, op.op)].append(i)

        for i, op in enumerate(schedule):
            if op.op in comm_types and get_peer(op) is not None and self.partner[i] < 0:
                for j in index.get((get_peer(op), op.mb_id, matching(op.op)), ()):
                    if get_peer(schedule[j]) == op.block_id and self.partner[j] < 0:
                        self.partner[i], self.partner[j] = j, i
                        break
        for i, op in enumerate(schedule):
            dep_type = _CHAIN.get(op.op)
            if dep_type is None:
                continue
            for j in index.get((op.block_id, op.mb_id, dep_type), ()):
                self._need(i, j)
                if schedule[j].op in recv_types and self.partner[j] >= 0:
                    self._need(i, self.partner[j])  # data exists only once the send is issued
        last_anchor: Dict[int, int] = {}
        self.ranks: List[int] = sorted({op.rank for op in schedule})
        self.by_rank: Dict[int, List[int]] = {r: [] for r in self.ranks}
        for i, op in enumerate(schedule):
            self.by_rank[op.rank].append(i)
            if op.op in _ANCHORED:
                if op.rank in last_anchor:
                    self._need(i, last_anchor[op.rank])
                last_anchor[op.rank] = i

    def _need(self, user: int, dep: int) -> None:
        self.users[dep].append(user)
        self.unmet[user] += 1

    def ready(self, i: int) -> bool:
        if self.emitted[i] or self.unmet[i]:
            return False
        j = self.partner[i]
        return j < 0 or self.emitted[j] or self.unmet[j] == 0

    def complete(self, i: int) -> None:
        for u in self.users[i]:
            self.unmet[u] -= 1

    def is_instant(self, i: int) -> bool:
        """Ops that take no pipeline slot: loss ops, all-reduce, prefetch, peerless comms."""
        op = self.ops[i]
        if op.op in compute_types:
            return False
        return op.op not in comm_types or self.partner[i] < 0

    def stuck_report(self) -> str:
        pending = [self.ops[i] for i in range(len(self.ops)) if not self.emitted[i]]
        return f"{len(pending)} ops can never become ready, e.g. {pending[:6]}"


def schedule_to_graph(schedule: List[Operation]) -> DirectedGraph:
    """Dependency graph in the reference's convention: an edge ``i → j`` means op ``i``
    depends on op ``j``; a matched send/recv pair is linked in both directions."""
    plan = _Plan(schedule)
    g = DirectedGraph(len(schedule))
    for dep, users in enumerate(plan.users):
        for u in users:
            # the "consumer waits for the sender" edges are implied by the pair link
            if schedule[dep].op in send_types and schedule[u].op in (T.FORWARD, T.BACKWARD_INPUTS):
                continue
            g.add_edge(u, dep)
    for i, j in enumerate(plan.partner):
        if j >= 0:
            g.add_edge(i, j)
    return g


# ---------------------------------------------------------------------------------------
# emission policies
# ---------------------------------------------------------------------------------------


def topological_sort(schedule: List[Operation]) -> List[Operation]:
    """Plain Kahn order (earliest original position first); each matched pair is emitted
    send-then-recv, adjacent.  No overlap optimisation."""
    plan = _Plan(schedule)
    heap = [i for i in range(len(schedule)) if plan.ready(i)]
    heapq.heapify(heap)
    queued = set(heap)
    out: List[Operation] = []

    def push_ready(cands):
        for c in cands:
            if c not in queued and plan.ready(c):
                queued.add(c)
                heapq.heappush(heap, c)

    def emit(i):
        plan.emitted[i] = True
        out.append(schedule[i])
        plan.complete(i)
        push_ready(plan.users[i])
        for u in plan.users[i]:
            if plan.partner[u] >= 0:
                push_ready([plan.partner[u]])

    while heap:
        i = heapq.heappop(heap)
        if plan.emitted[i]:
            continue
        j = plan.partner[i]
        if j >= 0 and not plan.emitted[j]:
            first, second = (i, j) if schedule[i].op in send_types else (j, i)
            emit(first)
            emit(second)
        else:
            emit(i)
    if len(out) != len(schedule):
        raise RuntimeError("schedule has a dependency cycle: " + plan.stuck_report())
    return out


def _rounds(schedule: List[Operation], pairs_first: bool) -> List[Operation]:
    plan = _Plan(schedule)
    ops = plan.ops
    pending: Dict[int, Dict[str, List[int]]] = {}
    for r in plan.ranks:
        q = {"instant": [], "recv": [], "compute": [], "send": []}
        for i in plan.by_rank[r]:
            if plan.is_instant(i):
                q["instant"].append(i)
            elif ops[i].op in recv_types:
                q["recv"].append(i)
            elif ops[i].op in send_types:
                q["send"].append(i)
            else:
                q["compute"].append(i)
        pending[r] = q
    out: List[Operation] = []

    def emit(i, now=True):
        plan.emitted[i] = True
        out.append(ops[i])
        if now:
            plan.complete(i)

    def take_first_ready(queue: List[int]) -> Optional[int]:
        for pos, i in enumerate(queue):
            if plan.ready(i):
                del queue[pos]
                return i
        return None

    def flush_instants(r) -> bool:
        any_emitted = False
        while True:
            i = take_first_ready(pending[r]["instant"])
            if i is None:
                return any_emitted
            emit(i)
            any_emitted = True

    total = len(ops)
    while len(out) < total:
        before = len(out)
        deferred: List[int] = []
        if pairs_first:
            # every transfer whose two ends are ready happens now, send next to recv
            for r in plan.ranks:
                while True:
                    i = take_first_ready(pending[r]["send"])
                    if i is None:
                        break
                    j = plan.partner[i]
                    pending[ops[j].rank]["recv"].remove(j)
                    emit(i)
                    emit(j)
        for r in plan.ranks:
            flush_instants(r)
            if not pairs_first:
                i = take_first_ready(pending[r]["recv"])
                if i is not None:
                    emit(i, now=False)
                    deferred.append(i)
            comp = pending[r]["compute"]
            if comp and plan.ready(comp[0]):
                emit(comp.pop(0))
                flush_instants(r)
            if not pairs_first:
                i = take_first_ready(pending[r]["send"])
                if i is not None:
                    emit(i, now=False)
                    deferred.append(i)
        for i in deferred:
            plan.complete(i)
        if len(out) == before:
            raise RuntimeError("comm scheduling cannot make progress: " + plan.stuck_report())
    return out


def smart_topological_sort(schedule: List[Operation]) -> List[Operation]:
    """Lock-step simulation: each round first performs every transfer whose two ends are
    ready (on all ranks at once), then lets every rank run one compute op."""
    return _rounds(schedule, pairs_first=True)


def pipelined_topological_sort(schedule: List[Operation]) -> List[Operation]:
    """Default policy.  Per round and rank: flush bookkeeping ops, **post the next ready
    recv**, run one compute op, **issue the next ready send**; transfers count as done at
    the end of the round.  The recv for the next micro-batch is therefore in flight while
    the current one computes, and a send leaves right after the op that produced it."""
    return _rounds(schedule, pairs_first=False)
