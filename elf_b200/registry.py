"""Plugin registries: schedulers, partitioners, tracers and comm schedulers.

Same surface as the reference's ``elf/registry.py:32-144`` (``register/get/get_key/
get_description/available``, membership, iteration, ``resolve``), rebuilt around a
single ``_Entry`` record per registered object so that aliases share one record
instead of living in two parallel dictionaries.

>>> from elf_b200.registry import SCHEDULERS
>>> SCHEDULERS.register("mine", lambda placement, nmb: [], "does nothing")
>>> Pipeline(model, sample, scheduler="mine")
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Callable, Dict, Generic, Iterable, Iterator, List, Protocol, TypeVar

__all__ = [
    "Registry",
    "SCHEDULERS",
    "PARTITIONERS",
    "TRACERS",
    "COMM_SCHEDULERS",
    "resolve",
    "SchedulerFn",
    "PartitionerFn",
    "TracerFn",
    "CommSchedulerFn",
]

T = TypeVar("T")


class SchedulerFn(Protocol):
    """``(placement, n_micro_batches) -> List[Operation]`` for *all* ranks
    (reference ``elf/registry.py:147-163``)."""

    def __call__(self, placement: List[int], n_micro_batches: int) -> list: ...


class PartitionerFn(Protocol):
    """``(graph, times, memories, n) -> List[List[fx.Node]]``
    (reference ``elf/registry.py:170-193``)."""

    def __call__(self, graph: Any, times: Dict, memories: Dict, n: int) -> list: ...


class TracerFn(Protocol):
    """``(model, sample) -> fx.GraphModule`` (reference ``elf/registry.py:199-217``)."""

    def __call__(self, model: Any, sample: Any) -> Any: ...


class CommSchedulerFn(Protocol):
    """``(schedule) -> schedule`` reordered so that p2p cannot deadlock
    (reference ``elf/registry.py:223-236``)."""

    def __call__(self, schedule: list) -> list: ...


@dataclass
class _Entry(Generic[T]):
    obj: T
    description: str
    keys: List[str] = field(default_factory=list)


class Registry(Generic[T]):
    """Name → object table with aliases."""

    def __init__(self, name: str):
        self._name = name
        self._by_key: Dict[str, _Entry[T]] = {}

    # -- registration ---------------------------------------------------
    def register(self, key: str | Iterable[str], obj: T, description: str = "") -> T:
        keys = [key] if isinstance(key, str) else list(key)
        for k in keys:
            held = self._by_key.get(k)
            if held is not None and held.obj is not obj:
                raise KeyError(f"{self._name} '{k}' already registered with a different object")
        entry = next((e for e in self._by_key.values() if e.obj is obj), None)
        if entry is None:
            entry = _Entry(obj, description)
        elif description:
            entry.description = description
        for k in keys:
            if k not in entry.keys:
                entry.keys.append(k)
            self._by_key[k] = entry
        return obj

    def unregister(self, key: str) -> None:
        entry = self._by_key.pop(key)
        entry.keys.remove(key)

    # -- lookup -----------------------------------------------------------
    def _entry(self, key: str) -> _Entry[T]:
        try:
            return self._by_key[key]
        except KeyError as exc:
            known = ", ".join(sorted(self._by_key)) or "<empty>"
            raise KeyError(f"Unknown {self._name} '{key}'. Available {self._name}s: [{known}]") from exc

    def get(self, key: str) -> T:
        return self._entry(key).obj

    def get_key(self, obj: T) -> str:
        for entry in self._by_key.values():
            if entry.obj is obj:
                return entry.keys[0]
        raise ValueError(f"Object {obj!r} not found in {self._name} registry")

    def get_description(self, key: str) -> str:
        return self._entry(key).description

    def available(self) -> List[str]:
        """One key per distinct object (the alphabetically first alias), sorted."""
        seen, out = set(), []
        for k in sorted(self._by_key):
            ident = id(self._by_key[k])
            if ident not in seen:
                seen.add(ident)
                out.append(k)
        return out

    def __contains__(self, key: object) -> bool:
        return isinstance(key, str) and key in self._by_key

    def __iter__(self) -> Iterator[str]:
        return iter(self._by_key)

    def __len__(self) -> int:
        return len(self._by_key)

    def __getitem__(self, key: str) -> T:
        return self.get(key)

    def __repr__(self) -> str:
        return f"<Registry[{self._name}] ({len(self)} items): {', '.join(sorted(self._by_key))}>"


SCHEDULERS: Registry[SchedulerFn] = Registry("scheduler")
PARTITIONERS: Registry[PartitionerFn] = Registry("partitioner")
TRACERS: Registry[TracerFn] = Registry("tracer")
COMM_SCHEDULERS: Registry[CommSchedulerFn] = Registry("comm_scheduler")


def resolve(var: str | Callable, registry: Registry) -> Callable:
    """Turn a registry key into its callable; callables pass through."""
    if callable(var):
        return var
    if var in registry:
        return registry[var]
    lines = [f"Unknown {registry._name} '{var}'. Available ones:"]
    lines += [f"\t{k}: {registry.get_description(k)}" for k in registry.available()]
    raise ValueError("\n".join(lines))
