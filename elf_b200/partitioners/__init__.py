"""Graph front-end: tracing → per-node profiling → partitioning → stage modules."""

from ..registry import PARTITIONERS, TRACERS
from .signature import Signature, sequential_signatures, signatures_from_sources_targets
from .tracing import extract_graph_export, extract_graph_fx, extract_graph_fx_safe, trace, try_extract_graph
from .profile import profile_operations
from .custom import split_graph, split_graph_constrained
from .dag import split_graph_min_volume
from .metis import split_graph_metis
from .dagP import split_graph_dagP
from .partition import PartitionResult, partition, split
from .utils import remove_inplace_leaves, prune_graph

PARTITIONERS.register("naive", split_graph, "Greedy prefix cuts balancing profiled time")
PARTITIONERS.register("constrained", split_graph_constrained, "Time-balanced cuts crossing as few tensors as possible (default)")
PARTITIONERS.register("metis", split_graph_metis, "gpmetis (volume objective) or the in-tree minimum-volume partitioner")
PARTITIONERS.register("dagP", split_graph_dagP, "rMLGP acyclic partitioner or the in-tree acyclic minimum-volume partitioner")

TRACERS.register("fx", extract_graph_fx, "torch.fx symbolic trace (split-backward and fused modules stay leaves)")
TRACERS.register("fx_safe", extract_graph_fx_safe, "torch.fx with untraceable sub-module classes turned into leaves")
TRACERS.register("export", extract_graph_export, "torch.export (non-strict)")
TRACERS.register("default", try_extract_graph, "fx, then fx_safe, then the other tracers")

__all__ = [
    "partition",
    "trace",
    "split",
    "profile_operations",
    "PartitionResult",
    "Signature",
    "sequential_signatures",
    "signatures_from_sources_targets",
    "remove_inplace_leaves",
    "prune_graph",
]
