from .adamw import FusedAdamW, DummyOptimizer, MixedPrecisionOptimizer
from .flat import FlatGroup, flatten_parameters

__all__ = ["FusedAdamW", "DummyOptimizer", "MixedPrecisionOptimizer", "FlatGroup", "flatten_parameters"]
