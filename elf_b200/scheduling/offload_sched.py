"""Scheduler wrappers that add activation offload to any base schedule.

In the reference this lives in the benchmark helpers only
(``benchmarks/benchmark_utils.py:338-407``); here it is part of the package so that the ILP
(``elf_b200/scheduling/ilp.py``) can emit the same ops.
"""

from __future__ import annotations

from typing import Callable, List, Set, Tuple

from ..registry import SCHEDULERS, resolve
from .scheduling import Operation, OperationType, OpOptions, compute_types, per_rank_programs

__all__ = ["offload_every", "apply_offload"]

T = OperationType


def apply_offload(schedule: List[Operation], chosen: Set[Tuple[int, int]], prefetching_time: int = 1) -> List[Operation]:
    """Mark the (stage, micro-batch) pairs in ``chosen``: their F and B carry
    ``ACTIVATION_OFFLOAD`` and a ``PREFETCH_ACTIVATIONS`` op is inserted
    ``prefetching_time`` compute ops ahead of the B in the rank's program."""
    out: List[Operation] = []
    for rank, prog in per_rank_programs(schedule).items():
        prog = list(prog)
        for op in prog:
            if op.op in (T.FORWARD, T.BACKWARD_INPUTS) and (op.block_id, op.mb_id) in chosen:
                op.options[OpOptions.ACTIVATION_OFFLOAD] = True
        inserts = []
        for idx, op in enumerate(prog):
            if op.op is T.BACKWARD_INPUTS and (op.block_id, op.mb_id) in chosen:
                pos, seen = idx, 0
                while pos > 0 and seen < prefetching_time:
                    pos -= 1
                    if prog[pos].op in compute_types:
                        seen += 1
                    if prog[pos].op is T.FORWARD and prog[pos].block_id == op.block_id and prog[pos].mb_id == op.mb_id:
                        pos += 1  # never before the forward that produces the activations
                        break
                # stay behind a LOSS_BACKWARD / comm ops glued in front of the B
                inserts.append((pos, Operation(op.block_id, op.mb_id, T.PREFETCH_ACTIVATIONS, rank)))
        for pos, new in sorted(inserts, key=lambda t: -t[0]):
            prog.insert(pos, new)
        out.extend(prog)
    return out


def offload_every(scheduler, ratio: int, prefetching_time: int = 1) -> Callable:
    base = resolve(scheduler, SCHEDULERS)
    ratio = max(1, int(ratio))

    def wrapped(placement, n_micro_batches):
        schedule = base(placement, n_micro_batches)
        chosen = {(op.block_id, op.mb_id) for op in schedule if op.op is T.FORWARD and op.mb_id % ratio == 0}
        return apply_offload(schedule, chosen, prefetching_time)

    return wrapped
