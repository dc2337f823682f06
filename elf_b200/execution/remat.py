"""Selective rematerialisation of sub-modules during a stage forward.

``RematManager.apply_selective_remat(strategy, mb)`` checkpoints every sub-module for
which ``strategy(name, module)`` is true (``name == ""`` is the whole stage) for the
duration of one forward, as the reference does (``elf/execution/remat.py:26-74``).  After
the forward, the W-pass inputs stashed by split-backward layers inside checkpointed
modules are dropped — the checkpoint re-run during B stashes them again — except stage
inputs, which no recomputation regenerates.
"""

from __future__ import annotations

import functools
from contextlib import contextmanager
from typing import Callable, List, Tuple

import torch
from torch.utils.checkpoint import CheckpointPolicy, checkpoint, create_selective_checkpoint_contexts

from ..zb_utils import LayerDW

__all__ = ["RematManager", "recompute_all_context_fn"]


class RematManager:
    def __init__(self, block):
        self.block = block

    def apply_selective_remat(self, remat_strategy: Callable, mb_id: int):
        @contextmanager
        def scope():
            chosen: List[Tuple[torch.nn.Module, Callable, bool]] = []
            for name, module in self.block.model.named_modules():
                if remat_strategy(name, module):
                    original = module.forward

                    # non-reentrant checkpointing also works when no input requires grad
                    def checkpointed(*args, __orig=original, **kwargs):
                        return checkpoint(__orig, *args, use_reentrant=False, **kwargs)

                    chosen.append((module, original, "forward" in module.__dict__))
                    module.forward = checkpointed
            try:
                yield
            finally:
                for module, original, was_instance_attr in chosen:
                    for sub in module.modules():
                        if not isinstance(sub, LayerDW):
                            continue
                        slots = sub.ctx["input"]
                        if len(slots) > mb_id and slots[mb_id] is not None and not getattr(slots[mb_id], "is_model_input", False):
                            sub.delete("input", mb_id)
                    if was_instance_attr:
                        module.forward = original
                    else:
                        del module.__dict__["forward"]  # back to the class's method

        return scope()


def recompute_all_context_fn():
    """``context_fn`` for ``torch.utils.checkpoint`` that forces every op to be recomputed."""

    def policy(*_args, **_kwargs):
        return CheckpointPolicy.MUST_RECOMPUTE

    return functools.partial(create_selective_checkpoint_contexts, policy)
