"""Stage signatures: which tensors a stage takes and returns, and which stages they link.

Same data model as the reference (``elf/partitioners/utils.py:26-146``): ``sources[i]`` is
the block id producing input ``i`` (``None`` = pipeline input), ``targets[j]`` the list of
block ids consuming output ``j`` (``None`` = pipeline output).
"""

from __future__ import annotations

from typing import Dict, Iterable, List, Optional, Sequence

__all__ = [
    "Signature",
    "signatures_from_sources_targets",
    "get_sources_targets_sequential",
    "sequential_signatures",
    "remove_dupes",
]


def remove_dupes(seq: Iterable) -> list:
    """Order-preserving de-duplication."""
    return list(dict.fromkeys(seq))


class Signature:
    def __init__(self, inputs: Sequence[str], outputs: Sequence[str], sources: Sequence[Optional[int]], targets: Sequence[List[Optional[int]]]):
        self.inputs = list(inputs)
        self.outputs = list(outputs)
        self.sources = list(sources)
        self.targets = [list(t) for t in targets]
        assert len(self.sources) == len(self.inputs), "one source per input"
        assert len(self.targets) == len(self.outputs), "one target list per output"

    @property
    def ninputs(self) -> int:
        return len(self.inputs)

    @property
    def noutputs(self) -> int:
        return len(self.outputs)

    def get_all_sources(self) -> list:
        """Distinct producer blocks, in input order."""
        return remove_dupes(self.sources)

    def get_all_targets(self) -> list:
        """Distinct consumer blocks, in output order."""
        return remove_dupes(t for tgt in self.targets for t in tgt)

    def __repr__(self) -> str:
        ins = ", ".join(f"{i} ({s})" for i, s in zip(self.inputs, self.sources))
        outs = ", ".join(f"{o} ({t})" for o, t in zip(self.outputs, self.targets))
        return f"Signature({ins}) -> ({outs})"

    __str__ = __repr__

    def __eq__(self, other) -> bool:
        return (
            isinstance(other, Signature)
            and (self.inputs, self.outputs, self.sources, self.targets)
            == (other.inputs, other.outputs, other.sources, other.targets)
        )


def signatures_from_sources_targets(sources: Dict[int, Dict[str, Optional[int]]], targets: Dict[int, Dict[str, list]]) -> List[Signature]:
    """``sources[i] = {input name: producer block}``, ``targets[i] = {output name: [consumer blocks]}``;
    names are sorted, as in the reference."""
    assert len(sources) == len(targets), "Sources and targets must have the same length"
    sigs = []
    for i in range(len(sources)):
        ins, outs = sorted(sources[i]), sorted(targets[i])
        sigs.append(Signature(ins, outs, [sources[i][k] for k in ins], [targets[i][k] for k in outs]))
    return sigs


def get_sources_targets_sequential(placement):
    n = len(placement)
    sources = {i: {"input": i - 1 if i else None} for i in range(n)}
    targets = {i: {"output": [i + 1 if i != n - 1 else None]} for i in range(n)}
    return sources, targets


def sequential_signatures(placement) -> List[Signature]:
    """Chain without skip connections: stage ``i`` reads ``input`` from ``i-1`` and sends
    ``output`` to ``i+1``.  For use with ``partitioner=False``."""
    return signatures_from_sources_targets(*get_sources_targets_sequential(placement))
