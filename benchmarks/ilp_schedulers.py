"""Replay an ILP solution computed offline (counterpart of the reference's
``benchmarks/ilp_schedulers.py``): the solution's ``order`` drives a ``FixedSchedule`` and its
remat tables are applied on top; ``selective_fwd`` checkpoints attention modules only."""

from __future__ import annotations

import json

from elf_b200.scheduling.ilp import RematScheduler as _RematScheduler
from elf_b200.scheduling.schedulers import FixedSchedule
from elf_b200.scheduling.scheduling import OperationType, OpOptions

__all__ = ["RematScheduler", "load_solution"]


def _attention_modules(name, module=None):
    return module is not None and "attention" in type(module).__name__.lower()


def load_solution(path: str) -> dict:
    with open(path) as f:
        return json.load(f)


class RematScheduler(_RematScheduler):
    def __init__(self, solution: dict):
        super().__init__(FixedSchedule({"order": solution["order"]}), solution)

    def __call__(self, placement, nmb):
        schedule = super().__call__(placement, nmb)
        selective = self.solution.get("selective_fwd") or []
        for op in schedule:
            if op.op is OperationType.FORWARD and selective:
                try:
                    if selective[op.block_id][op.mb_id]:
                        op.options[OpOptions.REMAT_STRATEGY] = _attention_modules
                except IndexError:
                    pass
        return schedule
