"""elf_b200 — Blackwell-native pipeline-parallel training.

Public surface mirrors the reference package (``elf/__init__.py:1-13``)."""

from .utils import Placement
from .partitioners.signature import sequential_signatures
from .zb_utils import replace_layer_with_layer_dw, replace_linear_with_linear_dw
from .pipeline import Pipeline, PipelineConfig

__version__ = "0.1.0"

__all__ = [
    "Pipeline",
    "PipelineConfig",
    "Placement",
    "sequential_signatures",
    "replace_layer_with_layer_dw",
    "replace_linear_with_linear_dw",
]
