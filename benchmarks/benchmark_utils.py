"""Shared pieces of the benchmark entry points: process-group start-up, clock sampling,
device timing, scheduler wrappers for checkpointing/offload, the ``bench`` harness and the
pipeline-vs-single-process correctness check (counterparts of the reference's
``benchmarks/benchmark_utils.py``)."""

from __future__ import annotations

import json
import os
import statistics
import subprocess
import threading
import time
from typing import Callable, Dict, List, Optional

import torch
import torch.distributed as dist

from elf_b200.scheduling.scheduling import Operation, OperationType, OpOptions, compute_types

__all__ = [
    "init_dist",
    "ClockSampler",
    "max_over_ranks",
    "get_checkpointed_scheduler",
    "get_offloaded_scheduler",
    "write_detailed_stats",
    "mem_state",
]


def init_dist(backend: Optional[str] = None):
    """Start ``torch.distributed`` from torchrun / mpirun / srun environment variables.
    Returns ``(local_rank, rank, world_size)``; with a world of one nothing is initialised."""
    env = os.environ
    rank = int(env.get("RANK", env.get("OMPI_COMM_WORLD_RANK", env.get("SLURM_PROCID", 0))))
    world = int(env.get("WORLD_SIZE", env.get("OMPI_COMM_WORLD_SIZE", env.get("SLURM_NTASKS", 1))))
    local = int(env.get("LOCAL_RANK", env.get("OMPI_COMM_WORLD_LOCAL_RANK", env.get("SLURM_LOCALID", rank))))
    use_cuda = torch.cuda.is_available()
    if use_cuda:
        torch.cuda.set_device(local % torch.cuda.device_count())
    if world > 1 and not dist.is_initialized():
        env.setdefault("MASTER_ADDR", "127.0.0.1")
        env.setdefault("MASTER_PORT", "29500")
        backend = backend or ("nccl" if use_cuda else "gloo")
        kwargs = {"device_id": torch.device("cuda", torch.cuda.current_device())} if backend == "nccl" else {}
        dist.init_process_group(backend, rank=rank, world_size=world, **kwargs)
    return local, rank, world


def max_over_ranks(value: float, device) -> float:
    if dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1:
        t = torch.tensor([value], dtype=torch.float64, device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())
    return float(value)


class ClockSampler:
    """Samples SM clocks and throttle reasons of one GPU with ``nvidia-smi`` while a timed
    region runs (read-only queries; nothing on the GPU is changed)."""

    FIELDS = "clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap"

    def __init__(self, gpu_index: int = 0, period_ms: int = 200):
        self.gpu_index, self.period_ms = gpu_index, period_ms
        self.proc = None
        self.lines: List[str] = []
        self._reader = None

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-i", str(self.gpu_index), "-lms", str(self.period_ms)],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True,
            )
            self._reader = threading.Thread(target=self._pump, daemon=True)
            self._reader.start()
        except (OSError, FileNotFoundError):
            self.proc = None
        return self

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def __exit__(self, *exc):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()
        return False

    def summary(self) -> Dict:
        sm, smax, power = [], [], []
        reasons = set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 7:
                continue
            try:
                sm.append(float(parts[0]))
                smax.append(float(parts[1]))
                power.append(float(parts[2]))
            except ValueError:
                continue
            for name, flag in zip(names, parts[3:7]):
                if flag.lower().startswith("active"):
                    reasons.add(name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["unavailable"], "samples": 0}
        # samples under load draw real power; idle samples at the start/end are dropped
        busy = [c for c, p in zip(sm, power) if p >= 0.5 * max(power)] or sm
        return {"sm_mhz": statistics.median(busy), "sm_max_mhz": max(smax), "power_w_max": max(power), "reasons": sorted(reasons), "samples": len(sm)}


def mem_state(device=None) -> Dict[str, float]:
    if not torch.cuda.is_available():
        return {}
    return {
        "allocated_gb": torch.cuda.memory_allocated(device) / 2**30,
        "peak_gb": torch.cuda.max_memory_allocated(device) / 2**30,
        "reserved_gb": torch.cuda.memory_reserved(device) / 2**30,
    }


def write_detailed_stats(path: str, detailed_stats: Dict, rank: int, world: int) -> None:
    """Merge every rank's ``detailed_stats`` into one JSON file, ranks taking turns."""
    for r in range(world):
        if r == rank:
            data = {}
            if os.path.exists(path) and r > 0:
                with open(path) as f:
                    data = json.load(f)
            data[str(rank)] = {k: dict(v) for k, v in detailed_stats.items()}
            with open(path, "w") as f:
                json.dump(data, f)
        if world > 1:
            dist.barrier()


# ---------------------------------------------------------------------------------------
# scheduler wrappers
# ---------------------------------------------------------------------------------------


def _whole_stage(name, _module=None):
    return name == ""


def _attention_only(name, module=None):
    return module is not None and "attention" in type(module).__name__.lower()


def _layer_wise(name, module=None):
    return module is not None and "decoderlayer" in type(module).__name__.lower()


def get_checkpointed_scheduler(scheduler, mode: str) -> Callable:
    """Wrap a scheduler so that forwards are checkpointed: ``full`` = the whole stage,
    ``simple`` = every decoder layer, ``selective`` = attention modules only."""
    from elf_b200.registry import SCHEDULERS, resolve

    base = resolve(scheduler, SCHEDULERS)
    strategy = {"full": _whole_stage, "simple": _layer_wise, "selective": _attention_only}[mode]

    def wrapped(placement, n_micro_batches):
        schedule = base(placement, n_micro_batches)
        last_rank = placement[-1]
        for op in schedule:
            if op.op is OperationType.FORWARD and not (mode == "full" and op.rank == last_rank and op.block_id == len(placement) - 1):
                op.options[OpOptions.REMAT_STRATEGY] = strategy
        return schedule

    return wrapped


def get_offloaded_scheduler(scheduler, ratio: int, prefetching_time: int = 1) -> Callable:
    """Wrap a scheduler so that every ``ratio``-th micro-batch keeps its activations in
    pinned host memory between F and B; the host→device copy is started
    ``prefetching_time`` compute ops before the B that needs it."""
    from elf_b200.scheduling.offload_sched import offload_every

    return offload_every(scheduler, ratio, prefetching_time)
