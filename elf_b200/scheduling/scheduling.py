"""Operation IR of a pipeline schedule, its text form and sanity checks.

A schedule is a flat ``List[Operation]`` covering **all** pipeline ranks; only the
relative order of the operations of one rank is meaningful.  The vocabulary and
option names are those of the reference (``elf/scheduling/scheduling.py:12-127``) so
that user-written schedulers keep working.  Unlike the reference, ``Operation.__eq__``
and ``__hash__`` agree (both include ``block_id``).
"""

from __future__ import annotations

import logging
from collections import defaultdict
from enum import Enum, StrEnum, auto
from typing import Dict, Iterable, List, Optional

logger = logging.getLogger("scheduling")

__all__ = [
    "OperationType",
    "OpOptions",
    "Operation",
    "comm_types",
    "compute_types",
    "recv_types",
    "send_types",
    "matching",
    "get_peer",
    "get_peer_rank",
    "schedule_to_str",
    "check_schedule_validity",
    "per_rank_programs",
]


class OperationType(Enum):
    RECV_FORWARD = 0
    FORWARD = 1
    SEND_FORWARD = 2
    RECV_BACKWARD = 3
    BACKWARD_INPUTS = 4
    BACKWARD_PARAMS = 5
    SEND_BACKWARD = 6
    LOSS_FORWARD = 7
    LOSS_BACKWARD = 8
    ALL_REDUCE_PARAM_GRADS = 9
    RECOMPUTE_FORWARD = 10
    RECOMPUTE_BACKWARD_INPUTS = 11
    PREFETCH_ACTIVATIONS = 12

    def __repr__(self) -> str:
        return self.name.lower()

    __str__ = __repr__


T = OperationType

recv_types = {T.RECV_FORWARD, T.RECV_BACKWARD}
send_types = {T.SEND_FORWARD, T.SEND_BACKWARD}
comm_types = recv_types | send_types
compute_types = {
    T.FORWARD,
    T.BACKWARD_INPUTS,
    T.BACKWARD_PARAMS,
    T.RECOMPUTE_FORWARD,
    T.RECOMPUTE_BACKWARD_INPUTS,
}


class OpOptions(StrEnum):
    """Keys of ``Operation.options`` understood by the runtime.

    REMAT_STRATEGY         ``(name, module) -> bool``: checkpoint these sub-modules in F.
    RECOMPUTE_ACTIVATIONS  on B: drop stashed layer inputs; a RECOMPUTE_FORWARD restores them before W.
    RECOMPUTE_GRADIENTS    on B: also drop stashed output-grads; RECOMPUTE_BACKWARD_INPUTS restores them.
    ACTIVATION_OFFLOAD     on F/B: saved tensors of this (stage, mb) live in pinned host memory.
    SAVE                   on RECOMPUTE_FORWARD: keep the autograd graph for a second backward.
    OFFLOAD_DW             on B: park the stashed W-pass operands of this (stage, mb) on the host until W.
    """

    REMAT_STRATEGY = auto()
    RECOMPUTE_ACTIVATIONS = auto()
    RECOMPUTE_GRADIENTS = auto()
    ACTIVATION_OFFLOAD = auto()
    SAVE = auto()
    OFFLOAD_DW = auto()


class Operation:
    """One unit of compute or communication: ``(block_id, mb_id, op, rank, **options)``.

    Communication ops name their peer **block** in ``options["src"]`` / ``options["dst"]``
    (``None`` = pipeline input/output, executed as a no-op)."""

    __slots__ = ("block_id", "mb_id", "op", "rank", "options")

    def __init__(self, block_id: int, mb_id: Optional[int], op: OperationType, rank: int, **options):
        self.block_id = block_id
        self.mb_id = mb_id
        self.op = op
        self.rank = rank
        self.options = options

    def key(self):
        return (self.block_id, self.mb_id, self.op, self.rank, get_peer(self))

    def __eq__(self, other: object) -> bool:
        return (
            isinstance(other, Operation)
            and other.block_id == self.block_id
            and other.op == self.op
            and other.mb_id == self.mb_id
            and other.rank == self.rank
            and other.options == self.options
        )

    def __hash__(self) -> int:
        return hash((self.block_id, self.mb_id, self.rank, self.op))

    def __repr__(self) -> str:
        return f"[Block {self.block_id}, mb {self.mb_id}]:{self.op!r}({self.options})"

    __str__ = __repr__

    def copy(self, **changes) -> "Operation":
        new = Operation(self.block_id, self.mb_id, self.op, self.rank, **dict(self.options))
        for k, v in changes.items():
            setattr(new, k, v)
        return new


_MATCH = {
    T.RECV_FORWARD: T.SEND_FORWARD,
    T.SEND_FORWARD: T.RECV_FORWARD,
    T.RECV_BACKWARD: T.SEND_BACKWARD,
    T.SEND_BACKWARD: T.RECV_BACKWARD,
}


def matching(op_type: OperationType) -> OperationType:
    """The other end of a transfer: recv(forward) ↔ send(forward), same for backward."""
    return _MATCH[op_type]


def get_peer(op: Operation):
    """Peer block id of a communication op (``None`` for pseudo-comms and non-comms)."""
    return op.options.get("dst", op.options.get("src", None))


def get_peer_rank(op: Operation, placement):
    peer = get_peer(op)
    return None if peer is None else placement[peer]


def per_rank_programs(schedule: Iterable[Operation]) -> Dict[int, List[Operation]]:
    """Split a global schedule into the ordered program of each rank."""
    progs: Dict[int, List[Operation]] = defaultdict(list)
    for op in schedule:
        progs[op.rank].append(op)
    return dict(sorted(progs.items()))


_LETTER = {
    T.RECV_FORWARD: "rf",
    T.FORWARD: "f",
    T.SEND_FORWARD: "sf",
    T.RECV_BACKWARD: "rb",
    T.BACKWARD_INPUTS: "b",
    T.BACKWARD_PARAMS: "w",
    T.SEND_BACKWARD: "sb",
    T.RECOMPUTE_FORWARD: "R",
    T.RECOMPUTE_BACKWARD_INPUTS: "R*",
    T.ALL_REDUCE_PARAM_GRADS: "(AR)",
    T.PREFETCH_ACTIVATIONS: "P",
}


def _token(op: Operation) -> str:
    letter = _LETTER[op.op]
    if op.op is T.FORWARD:
        rematted = (not op.options.get(OpOptions.SAVE, True)) or bool(op.options.get(OpOptions.REMAT_STRATEGY, False))
        letter = "F" if rematted else "f"
    elif op.op is T.BACKWARD_INPUTS:
        letter = {"full": "b", "gradients": "b*", "none": "B"}.get(op.options.get(OpOptions.SAVE, "full"), "b")
    mb = "" if op.mb_id is None else op.mb_id
    peer = f"({get_peer(op)})" if op.op in comm_types else ""
    return f"{letter}{op.block_id}-{mb}{peer}"


def schedule_to_str(schedule: List[Operation], print_comms: bool = False) -> str:
    """One line per rank: ``f``/``F`` forward (plain / rematerialised), ``b`` ``b*`` ``B``
    backward-inputs, ``w`` backward-params, ``R`` ``R*`` recomputes, ``(AR)``, ``P``
    prefetch; with ``print_comms`` also ``rf sf rb sb`` and the peer block in brackets.
    Loss ops are not shown."""
    lines = []
    for rank, ops in per_rank_programs(schedule).items():
        toks = [_token(op) for op in ops if op.op in _LETTER and (print_comms or op.op not in comm_types)]
        lines.append(f"Rank {rank}: {' '.join(toks)}")
    return "\n".join(lines)


def check_schedule_validity(schedule: List[Operation]) -> None:
    """Structural checks (reference ``elf/scheduling/scheduling.py:232-270``): every rank
    touches every micro-batch; per (stage, mb): F before B, a W exists iff a B does and is
    not before it.  Also checked here: recomputes sit between their B and their W."""
    all_mbs = {op.mb_id for op in schedule if op.mb_id is not None}
    for rank, ops in per_rank_programs(schedule).items():
        seen = {op.mb_id for op in ops if op.mb_id is not None}
        assert len(seen) == len(all_mbs), f"[Rank {rank}] has {len(seen)} microbatches, expected {len(all_mbs)}"
        first: Dict[tuple, int] = {}
        for pos, op in enumerate(ops):
            first.setdefault((op.block_id, op.mb_id, op.op), pos)
        for (block, mb, kind), pos in first.items():
            if mb is None:
                continue
            if kind is T.BACKWARD_INPUTS:
                f = first.get((block, mb, T.FORWARD))
                assert f is not None, f"[Rank {rank}] Forward should be present for microbatch {mb}"
                assert f < pos, f"[Rank {rank}] Forward should be before backward inputs for microbatch {mb}"
                w = first.get((block, mb, T.BACKWARD_PARAMS))
                assert w is not None, (
                    f"[Rank {rank}] Backward params should be present for microbatch {mb} since backward inputs is present"
                )
                assert pos <= w, f"[Rank {rank}] Backward params should be after backward inputs for microbatch {mb}"
            elif kind in (T.RECOMPUTE_FORWARD, T.RECOMPUTE_BACKWARD_INPUTS):
                b = first.get((block, mb, T.BACKWARD_INPUTS))
                w = first.get((block, mb, T.BACKWARD_PARAMS))
                assert b is not None and w is not None and b < pos < w, (
                    f"[Rank {rank}] {kind!r} of block {block}, microbatch {mb} must sit between its B and its W"
                )
            elif kind is T.BACKWARD_PARAMS:
                assert (block, mb, T.BACKWARD_INPUTS) in first, (
                    f"[Rank {rank}] Backward params without backward inputs for microbatch {mb}"
                )
