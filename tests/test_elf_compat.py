"""Code written against the reference's import paths runs on this package unchanged."""

import importlib

import pytest

# every import the reference's examples, benchmarks, tests and documentation use
IMPORTS = """
from elf import Pipeline, PipelineConfig, Placement, sequential_signatures, replace_layer_with_layer_dw
from elf.registry import SCHEDULERS, PARTITIONERS, TRACERS, COMM_SCHEDULERS, Registry, resolve
from elf.scheduling import Operation, OperationType, OpOptions, add_comms, schedule_to_str, check_schedule_validity
from elf.scheduling.scheduling import Operation, OpOptions, OperationType, compute_types
from elf.scheduling.schedulers import FixedSchedule
from elf.scheduling.ilp import profile, profile_stage, solve_remat, stagerematify, AutoScheduler, RematScheduler, profile_all_stages
from elf.scheduling.comm_scheduling import DirectedGraph
from elf.partitioners import partition, trace, split, profile_operations, PartitionResult, Signature, sequential_signatures
from elf.partitioners.utils import Signature, remove_inplace_leaves, signatures_from_sources_targets, sequential_signatures
from elf.zb_utils import LayerDW, LinearDW, Conv1dDW, replace_linear_with_linear_dw
from elf.execution import PipelineBlock, Engine
from elf.execution.block import PipelineBlock
from elf.execution.offload import OffloadToCPU, PinnedHostTensorPool
from elf.utils import Placement, Timer, TensorMetadata, send_models, recv_models, broadcast_models
from elf.pipeline import PipelineConfig
""".strip().splitlines()


@pytest.mark.parametrize("line", IMPORTS)
def test_reference_import_line(line):
    exec(line, {})


def test_both_spellings_share_their_objects():
    import elf
    import elf_b200

    assert elf.Pipeline is elf_b200.Pipeline
    assert importlib.import_module("elf.registry").SCHEDULERS is importlib.import_module("elf_b200.registry").SCHEDULERS
    assert importlib.import_module("elf.scheduling.ilp") is importlib.import_module("elf_b200.scheduling.ilp")
    assert set(elf.__all__) >= {"Pipeline", "PipelineConfig", "Placement", "sequential_signatures", "replace_layer_with_layer_dw"}


def test_reference_style_program_runs():
    """The manual-split example of the reference (``examples/basic_no_partition.py``), shrunk
    to a tiny MLP on CPU: same imports, same calls."""
    import torch
    import torch.nn as nn

    from elf import Pipeline, sequential_signatures
    from elf.zb_utils import replace_linear_with_linear_dw

    torch.manual_seed(0)
    parts = [nn.Sequential(nn.Linear(16, 32), nn.ReLU()), nn.Sequential(nn.Linear(32, 32), nn.ReLU()), nn.Sequential(nn.Linear(32, 8))]
    for part in parts:
        replace_linear_with_linear_dw(part, "cpu")
    placement = [0, 0, 0]
    pipe = Pipeline(parts, None, partitioner=False, placement=placement, signatures=sequential_signatures(placement), scheduler="afab")
    x, y = torch.randn(8, 16), torch.randn(8, 8)
    outputs, loss = pipe(x, y, nn.functional.mse_loss, split_size=2)
    assert len(outputs) == 4 and torch.isfinite(loss)
    assert all(p.grad is not None for p in pipe.parameters())
    pipe.zero_grad()
    pipe.clear()
