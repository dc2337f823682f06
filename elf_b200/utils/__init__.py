"""Utilities: placements, p2p metadata, timers, model shipping, FLOP formulas."""

from .placement import Placement
from .metadata import TensorMetadata, DTYPES
from .timers import Timer, TimerCPU, TimerGPU
from .shipping import send_models, recv_models, broadcast_models, transport_device
from .flops import prod, linear_flops, attention_flops, transformer_step_flops
from .misc import _is_mpi, pretty_print_params, NameMapping

dtypes = DTYPES

__all__ = [
    "Placement",
    "TensorMetadata",
    "Timer",
    "TimerCPU",
    "TimerGPU",
    "send_models",
    "recv_models",
    "broadcast_models",
    "transport_device",
    "prod",
    "pretty_print_params",
    "NameMapping",
    "linear_flops",
    "attention_flops",
    "transformer_step_flops",
]
