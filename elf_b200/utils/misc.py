"""Small helpers (reference ``elf/utils.py:34-47,223-246``)."""

from __future__ import annotations

import torch.distributed as dist

__all__ = ["_is_mpi", "pretty_print_params", "NameMapping"]


def _is_mpi() -> bool:
    return dist.is_available() and dist.is_initialized() and dist.get_backend() == dist.Backend.MPI


def pretty_print_params(n) -> str:
    if n > 1e9:
        return f"{n / 1e9:.1f}B"
    if n > 1e6:
        return f"{n / 1e6:.1f}M"
    return f"{int(n)}"


class NameMapping:
    """Two-way map between the input names of one block and the output names of another."""

    def __init__(self, inputs, outputs):
        self.inputs_to_outputs = dict(zip(inputs, outputs))
        self.outputs_to_inputs = dict(zip(outputs, inputs))

    def to_output(self, name):
        return self.inputs_to_outputs[name]

    def to_input(self, name):
        return self.outputs_to_inputs[name]

    def __repr__(self):
        body = "".join(f"  {i} <-> {o}\n" for i, o in self.inputs_to_outputs.items())
        return f"NameMapping: (\n{body})"
