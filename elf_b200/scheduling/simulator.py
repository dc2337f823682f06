"""Timeline simulation of a schedule: makespan, bubble, live-activation peak, deadlock check.

This is the oracle the tests use for every generator and comm scheduler, and the cost
model behind ``AutoScheduler``'s fallback ranking.  It has no counterpart in the
reference, whose only static guard is the back-edge assertion at the end of its
pipelined comm scheduler (``elf/scheduling/comm_scheduling.py:443-448``).

Two views are offered:

``simulate(schedule, ...)``
    data-flow timing.  Each rank executes its compute ops in program order; an op starts
    when the rank is free and its producers (previous stage's F, next stage's B, own B
    for W) have finished (+ ``hop`` across ranks).  Communication ops are ignored.

``replay_comms(schedule, placement)``
    protocol check for a schedule that contains comm ops.  Ranks step through their
    programs; sends and recvs are *posted* without blocking, a compute op blocks until
    every recv it consumes has been matched by a posted send, and on every channel
    (ordered block pair × direction; the runtime gives each its own communicator or tag
    space) the k-th send must be the k-th recv, which is how NCCL and gloo match p2p
    traffic.  Returns normally or raises ``DeadlockError``.
"""

from __future__ import annotations

from collections import defaultdict, deque
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple

from .scheduling import Operation, OperationType, get_peer, per_rank_programs, recv_types, send_types

__all__ = ["simulate", "SimResult", "replay_comms", "DeadlockError"]

T = OperationType


class DeadlockError(RuntimeError):
    pass


@dataclass
class SimResult:
    makespan: float
    busy: Dict[int, float]
    start: Dict[int, float]
    end: Dict[int, float]
    peak_live: Dict[int, int]
    spans: Dict[Tuple[int, int, OperationType], Tuple[float, float]] = field(repr=False, default_factory=dict)

    @property
    def bubble_fraction(self) -> float:
        """Idle share of the busiest-possible rectangle ``ranks × makespan``."""
        total = self.makespan * len(self.busy)
        return 0.0 if total == 0 else 1.0 - sum(self.busy.values()) / total

    def idle(self, rank: int) -> float:
        return self.makespan - self.busy[rank]


_DEFAULT_COST = {
    T.FORWARD: 1.0,
    T.BACKWARD_INPUTS: 1.0,
    T.BACKWARD_PARAMS: 1.0,
    T.RECOMPUTE_FORWARD: 1.0,
    T.RECOMPUTE_BACKWARD_INPUTS: 1.0,
}


def simulate(
    schedule: Sequence[Operation],
    placement: Optional[Sequence[int]] = None,
    cost=None,
    hop: float = 0.0,
) -> SimResult:
    """``cost`` is ``{OperationType: t}``, ``{(OperationType, stage): t}`` or a callable
    ``cost(op) -> t``; missing entries default to 1 for compute ops and 0 otherwise."""

    def duration(op: Operation) -> float:
        if callable(cost):
            return float(cost(op))
        if cost:
            if (op.op, op.block_id) in cost:
                return float(cost[(op.op, op.block_id)])
            if op.op in cost:
                return float(cost[op.op])
        return _DEFAULT_COST.get(op.op, 0.0)

    progs = {r: [op for op in ops if op.op not in recv_types and op.op not in send_types] for r, ops in per_rank_programs(schedule).items()}
    n_stages = 1 + max(op.block_id for op in schedule)
    rank_of = {}
    for op in schedule:
        rank_of[op.block_id] = op.rank
    if placement is not None:
        rank_of.update({s: r for s, r in enumerate(placement)})

    has_b = {(op.block_id, op.mb_id) for op in schedule if op.op is T.BACKWARD_INPUTS}
    end_of: Dict[Tuple[int, int, OperationType], float] = {}
    spans: Dict[Tuple[int, int, OperationType], Tuple[float, float]] = {}
    pc = {r: 0 for r in progs}
    free = {r: 0.0 for r in progs}
    busy = {r: 0.0 for r in progs}
    first = {}
    live = {r: 0 for r in progs}
    peak = {r: 0 for r in progs}

    def hop_between(a: int, b: int) -> float:
        return hop if rank_of.get(a) != rank_of.get(b) else 0.0

    def ready_time(op: Operation) -> Optional[float]:
        s, mb = op.block_id, op.mb_id
        deps = []
        if op.op is T.FORWARD and s > 0:
            deps.append(((s - 1, mb, T.FORWARD), hop_between(s - 1, s)))
        elif op.op is T.BACKWARD_INPUTS:
            deps.append(((s, mb, T.FORWARD), 0.0))
            if s < n_stages - 1 and (s + 1, mb) in has_b:
                deps.append(((s + 1, mb, T.BACKWARD_INPUTS), hop_between(s + 1, s)))
        elif op.op in (T.BACKWARD_PARAMS, T.RECOMPUTE_FORWARD, T.RECOMPUTE_BACKWARD_INPUTS):
            if (s, mb) in has_b:
                deps.append(((s, mb, T.BACKWARD_INPUTS), 0.0))
        t = 0.0
        for key, lag in deps:
            if key not in end_of:
                return None
            t = max(t, end_of[key] + lag)
        return t

    remaining = sum(len(p) for p in progs.values())
    while remaining:
        moved = False
        for r, prog in progs.items():
            while pc[r] < len(prog):
                op = prog[pc[r]]
                rt = ready_time(op)
                if rt is None:
                    break
                begin = max(free[r], rt)
                d = duration(op)
                finish = begin + d
                key = (op.block_id, op.mb_id, op.op)
                end_of[key] = finish
                spans[key] = (begin, finish)
                if d > 0:
                    first.setdefault(r, begin)
                    busy[r] += d
                free[r] = finish
                if op.op is T.FORWARD:
                    live[r] += 1
                    peak[r] = max(peak[r], live[r])
                elif op.op is T.BACKWARD_PARAMS:
                    live[r] -= 1
                pc[r] += 1
                remaining -= 1
                moved = True
        if not moved:
            stuck = {r: progs[r][pc[r]] for r in progs if pc[r] < len(progs[r])}
            raise DeadlockError(f"no rank can advance; waiting ops: {stuck}")
    makespan = max(free.values()) if free else 0.0
    return SimResult(makespan, busy, first, dict(free), peak, spans)


def replay_comms(schedule: Sequence[Operation], placement: Sequence[int]) -> int:
    """Protocol replay (see module docstring).  Returns the number of scheduling rounds."""
    progs = per_rank_programs(schedule)
    pc = {r: 0 for r in progs}
    # channel = (src_block, dst_block, "fwd"|"bwd") → FIFO of (src_block, dst_block, mb)
    posted_sends: Dict[tuple, deque] = defaultdict(deque)
    posted_recvs: Dict[tuple, deque] = defaultdict(deque)
    arrived = set()  # (dst_block, src_block, mb, dir) payloads matched
    local = set()  # same-rank hand-offs done
    computed = set()

    def direction(op):
        return "fwd" if op.op in (T.RECV_FORWARD, T.SEND_FORWARD) else "bwd"

    def match(chan):
        s, r = posted_sends[chan], posted_recvs[chan]
        while s and r:
            a, b = s.popleft(), r.popleft()
            if a != b:
                raise DeadlockError(f"channel {chan}: send {a} meets recv {b} (order mismatch)")
            arrived.add((b[1], b[0], b[2], chan[2]))

    needs: Dict[tuple, List[tuple]] = defaultdict(list)
    for op in schedule:
        if op.op in recv_types and get_peer(op) is not None:
            kind = T.FORWARD if op.op is T.RECV_FORWARD else T.BACKWARD_INPUTS
            needs[(op.block_id, op.mb_id, kind)].append((op.block_id, get_peer(op), op.mb_id, direction(op)))

    rounds = 0
    remaining = sum(len(p) for p in progs.values())
    while remaining:
        rounds += 1
        moved = False
        for r, prog in progs.items():
            while pc[r] < len(prog):
                op = prog[pc[r]]
                peer = get_peer(op)
                if op.op in send_types or op.op in recv_types:
                    if peer is not None:
                        d = direction(op)
                        if op.op in send_types:
                            produced = (op.block_id, op.mb_id, T.FORWARD if d == "fwd" else T.BACKWARD_INPUTS)
                            if produced not in computed:
                                raise DeadlockError(f"{op} is issued before its payload is computed")
                            if placement[peer] == r:
                                local.add((peer, op.block_id, op.mb_id, d))
                            else:
                                chan = (op.block_id, peer, d)
                                posted_sends[chan].append((op.block_id, peer, op.mb_id))
                                match(chan)
                        else:
                            if placement[peer] != r:
                                chan = (peer, op.block_id, d)
                                posted_recvs[chan].append((peer, op.block_id, op.mb_id))
                                match(chan)
                elif op.op in (T.FORWARD, T.BACKWARD_INPUTS):
                    want = needs.get((op.block_id, op.mb_id, op.op), [])
                    if not all((w in arrived) or (w in local) for w in want):
                        break
                    computed.add((op.block_id, op.mb_id, op.op))
                pc[r] += 1
                remaining -= 1
                moved = True
        if not moved:
            stuck = {r: progs[r][pc[r]] for r in progs if pc[r] < len(progs[r])}
            raise DeadlockError(f"deadlock: every rank is blocked; waiting ops: {stuck}")
    leftovers = {c: list(q) for c, q in list(posted_sends.items()) + list(posted_recvs.items()) if q}
    if leftovers:
        raise DeadlockError(f"unmatched p2p traffic: {leftovers}")
    return rounds
