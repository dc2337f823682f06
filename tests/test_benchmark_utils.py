"""The benchmark harness pieces: hand-made partitions, meta-device materialisation, the timing
loop and the pipeline-vs-single-process check (CPU, one process and gloo ranks)."""

import pytest
import torch

from benchmarks.benchmark_utils import balanced_partition, bench, check_correctness, get_handcrafted_partition, meta_to_device
from elf_b200 import Pipeline, replace_layer_with_layer_dw
from elf_b200.models.simple import FullTransformer
from tests.dist_utils import run_ranks

SMALL = dict(input_dim=64, hidden_dim=32, n_blocks=5, seq_len=16, num_heads=2, ffn_dim=64)


def test_balanced_partition_puts_the_remainder_in_the_middle_first():
    assert balanced_partition(8, [0, 1, 2, 3]) == [2, 2, 2, 2]
    assert balanced_partition(9, [0, 1, 2, 3]) == [2, 2, 3, 2]
    assert balanced_partition(10, [0, 1, 2, 3]) == [2, 3, 3, 2]
    assert balanced_partition(11, [0, 1, 2, 3]) == [3, 3, 3, 2]
    assert sum(balanced_partition(30, list(range(8)))) == 30


def test_meta_to_device_initialises_everything():
    with torch.device("meta"):
        model = FullTransformer(**SMALL)
    assert all(p.is_meta for p in model.parameters())
    meta_to_device(model, "cpu", seed=0)
    for name, p in model.named_parameters():
        assert not p.is_meta and torch.isfinite(p).all(), name
    assert float(model.head.weight.detach().std()) > 0
    out = model(model.get_sample(2))
    assert out.shape == (2, SMALL["seq_len"], SMALL["input_dim"])


def test_handcrafted_partition_and_bench_loop():
    with torch.device("meta"):
        model = FullTransformer(**SMALL)
    placement = [0, 0, 0]
    parts = get_handcrafted_partition(model, 0, placement, device="cpu")
    assert [sum(1 for m in p if type(m).__name__ == "TransformerBlock") for p in parts] == [2, 2, 1]
    assert isinstance(parts[0][0], torch.nn.Module) and parts[-1][-1] is model.head
    for p in parts:
        replace_layer_with_layer_dw(p)
    median, peaks, times = bench(model, parts, "afab", placement, nmb=2, ntrials=2, n_iterations=2, warmup=1, outputs="none")
    assert len(times) == 2 and median > 0 and peaks == [0.0]


def _correctness_worker(rank, world):
    torch.manual_seed(0)
    model = FullTransformer(**SMALL)
    replace_layer_with_layer_dw(model)
    sample = model.get_sample(1)
    pipe = Pipeline(model, sample, scheduler="1f1b", partitioner="constrained", outputs="device")
    report = check_correctness(model, pipe)
    if rank == pipe.placement[-1]:
        assert set(report) == {"output", "loss", "grad"} and report["grad"] < 1e-3
    pipe.clear()


@pytest.mark.dist
def test_check_correctness_two_ranks():
    run_ranks(_correctness_worker, 2)


def test_offline_memory_plan_fits_the_budget():
    """``benchmarks/plan_memory.py``: analytic stage statistics -> ILP.  A budget below the
    unconstrained peak must be met by recomputation at the price of a longer planned step."""
    from benchmarks.plan_memory import main as plan

    free = plan(["--name", "llama-1.3b", "--pp", "2", "--nmb", "8", "--scheduler", "zbv", "--memory-budget-gb", "1000", "--time-limit", "30"])
    assert free["slots"]["full_fwd"] + free["slots"]["activations_bwd"] + free["slots"]["full_bwd"] == 0
    budget = 0.9 * max(free["peak_gb_per_rank"])
    assert budget > max(free["resident_gb_per_rank"])
    tight = plan(["--name", "llama-1.3b", "--pp", "2", "--nmb", "8", "--scheduler", "zbv", "--memory-budget-gb", f"{budget:.3f}", "--time-limit", "30"])
    assert "infeasible" not in tight
    assert max(tight["peak_gb_per_rank"]) <= budget + 0.06  # rounded to 0.1 GB in the report
    assert sum(tight["slots"][k] for k in ("full_fwd", "activations_bwd", "full_bwd")) > 0
    assert tight["planned_step_ms"] >= free["planned_step_ms"]
    impossible = plan(["--name", "llama-1.3b", "--pp", "2", "--nmb", "8", "--scheduler", "zbv", "--memory-budget-gb", f"{0.5 * max(free['resident_gb_per_rank']):.3f}", "--time-limit", "10"])
    assert "infeasible" in impossible


def test_planned_solution_replays_through_the_benchmark_cli(tmp_path):
    """Plan offline (a budget that forces recomputation), store the solution, and train with it:
    ``run_transformer.py --scheduler file`` takes order, placement and remat tables from the file."""
    import json
    import os
    import subprocess
    import sys

    from benchmarks.plan_memory import main as plan

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    path = str(tmp_path / "plan.json")
    report = plan(["--name", "llama-tiny", "--pp", "2", "--nmb", "4", "--scheduler", "zbv", "--memory-budget-gb", "0.026", "--time-limit", "20", "--out", path])
    assert "infeasible" not in report and report["slots"]["full_fwd"] + report["slots"]["activations_bwd"] + report["slots"]["full_bwd"] > 0
    with open(path) as fh:
        stored = json.load(fh)
    assert stored["placement"] == [0, 1, 1, 0] and len(stored["order"]) == 3 * 4 * 4
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr", "127.0.0.1", "--master-port", "29773",
           os.path.join(root, "benchmarks", "run_transformer.py"), "--architecture", "llama", "--name", "llama-tiny", "--partitioner", "handcrafted",
           "--scheduler", "file", "--schedule-file", path, "--nmb", "4", "--mb-size", "1", "--niters", "2", "--warmup", "1", "--backend", "gloo"]
    out = subprocess.run(cmd, cwd=root, capture_output=True, text=True, timeout=300, env=dict(os.environ, CUDA_VISIBLE_DEVICES=""))
    assert out.returncode == 0, out.stdout[-1500:] + out.stderr[-3000:]
    assert "tokens_per_s" in out.stdout
