"""Stage → rank maps.

``Placement`` is a ``list`` of ranks indexed by stage id, as in the reference
(``elf/utils.py:50-147``).  Ranks stored here are *pipeline-local* (``0..pp-1``);
the data-parallel replica offset is applied by the runtime when it talks to
``torch.distributed``, never baked into the list handed to a scheduler.  (The
reference bakes the offset in, ``elf/pipeline.py:165-168``, which empties the 1F1B
schedule and breaks ZBV/Hanayo on every replica but the first.)
"""

from __future__ import annotations

from typing import Iterable, List

__all__ = ["Placement"]

_V_SHAPED = {"hanayo", "zbv"}
_INTERLEAVED = {"megatron"}


class Placement(List[int]):
    def __init__(self, placement: Iterable[int] = ()):
        super().__init__(int(r) for r in placement)
        if len(self) and min(self) < 0:
            raise ValueError("Placement ranks must be non-negative")
        try:
            import torch.distributed as dist

            if dist.is_available() and dist.is_initialized() and len(self):
                assert max(self) < dist.get_world_size(), "Placement is out of bounds"
        except ImportError:  # pragma: no cover
            pass

    # -- queries -------------------------------------------------------------
    def get_ids(self, rank: int) -> List[int]:
        """Stage ids hosted by ``rank``, ascending."""
        return [s for s, r in enumerate(self) if r == rank]

    @property
    def n_devices(self) -> int:
        return len(set(self))

    def ranks(self) -> List[int]:
        """Distinct ranks in order of first appearance."""
        return list(dict.fromkeys(self))

    def head(self) -> int:
        return self[0]

    def tail(self) -> int:
        return self[-1]

    def is_head(self, rank: int) -> bool:
        return rank == self[0]

    def is_tail(self, rank: int) -> bool:
        return rank == self[-1]

    # -- constructors ----------------------------------------------------------
    def add_offset(self, offset: int) -> "Placement":
        return Placement(r + offset for r in self)

    def normalised(self) -> "Placement":
        """Same pattern on ranks ``0..n-1`` (smallest rank becomes 0)."""
        base = min(self) if len(self) else 0
        return Placement(r - base for r in self)

    @staticmethod
    def linear(pp: int) -> "Placement":
        return Placement(range(pp))

    @staticmethod
    def interleaved(pp: int, chunks: int = 2) -> "Placement":
        return Placement(list(range(pp)) * chunks)

    @staticmethod
    def v_shape(pp: int, waves: int = 1) -> "Placement":
        return Placement((list(range(pp)) + list(reversed(range(pp)))) * waves)

    @staticmethod
    def default(scheduler, pp: int) -> "Placement":
        """Placement a scheduler expects when the user gives none: V for
        ``hanayo``/``zbv``, two interleaved chunks for ``megatron``, else linear."""
        name = "" if callable(scheduler) else str(scheduler)
        if name in _V_SHAPED:
            return Placement.v_shape(pp)
        if name in _INTERLEAVED:
            return Placement.interleaved(pp, 2)
        return Placement.linear(pp)

    def __mul__(self, n):  # keep the subclass through ``placement * interleaving``
        return Placement(list(self) * n)

    __rmul__ = __mul__
