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

from elf_b200.scheduling.scheduling import OperationType, OpOptions

__all__ = [
    "bench",
    "meta_to_device",
    "balanced_partition",
    "get_handcrafted_partition",
    "get_handcrafted_imbalanced_partition",
    "check_correctness",
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


# ---------------------------------------------------------------------------------------
# timing harness, hand-made partitions, pipeline-vs-single-process check
# ---------------------------------------------------------------------------------------


def meta_to_device(model: torch.nn.Module, device="cuda", std: float = 0.02, seed: Optional[int] = None) -> torch.nn.Module:
    """Materialise a module built under ``torch.device("meta")`` on ``device`` and initialise
    it: modules that define ``reset_parameters`` use it, remaining matrices get N(0, ``std``),
    remaining vectors their customary constant (1 for norm gains, 0 for biases).  The
    reference's helper of the same name (``benchmarks/benchmark_utils.py:146-152``) looks for
    ``reset_parameters`` on *parameters* and therefore leaves memory uninitialised."""
    if any(p.is_meta for p in model.parameters()) or any(b.is_meta for b in model.buffers()):
        model.to_empty(device=device)
    else:
        model.to(device)
    gen = torch.Generator(device="cpu")
    if seed is not None:
        gen.manual_seed(seed)
    done = set()
    for module in model.modules():
        reset = getattr(module, "reset_parameters", None)
        if callable(reset):
            reset()
            done.update(id(p) for p in module.parameters(recurse=False))
    with torch.no_grad():
        for name, p in model.named_parameters():
            if id(p) in done:
                continue
            if p.dim() >= 2:
                p.copy_(torch.empty(p.shape, dtype=torch.float32).normal_(0.0, std, generator=gen))
            elif name.endswith("bias"):
                p.zero_()
            else:
                p.fill_(1.0)
    return model


def balanced_partition(n: int, placement: List[int]) -> List[int]:
    """Blocks per stage for ``n`` equal blocks: the remainder goes to the middle stages first
    (from the back), then to the first stage; the last stage, which also carries the head, is
    served last (``benchmarks/benchmark_utils.py:155-172`` of the reference)."""
    k = len(placement)
    counts = [n // k] * k
    order = [k - i for i in range(2, k + 1)] + [k - 1]
    for i in order[: n % k]:
        counts[i] += 1
    return counts


def get_handcrafted_imbalanced_partition(model, rank: int, placement: List[int], factors: List[int], device=None) -> List[torch.nn.Module]:
    """Stages hosted by pipeline rank ``rank`` when stage ``i`` takes ``factors[i]`` consecutive
    entries of ``model.blocks``; ``model.embed`` joins the first stage, ``model.ln`` / ``model.head``
    the last.  The stages are materialised on ``device`` (default: this process's GPU, else CPU)."""
    blocks = list(model.blocks)
    assert sum(factors) == len(blocks), f"factors {factors} do not cover the {len(blocks)} blocks"
    assert len(factors) == len(placement)
    if device is None:
        device = torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else torch.device("cpu")
    stages, start = [], 0
    for i, n in enumerate(factors):
        mods = blocks[start : start + n]
        start += n
        if i == 0:
            mods = [m for m in (getattr(model, "embed", None),) if m is not None] + mods
        if i == len(factors) - 1:
            mods += [m for m in (getattr(model, "ln", None), getattr(model, "head", None)) if m is not None]
        stages.append(torch.nn.Sequential(*mods))
    mine = [s for s, r in zip(stages, placement) if r == rank]
    return [meta_to_device(s, device) for s in mine]


def get_handcrafted_partition(model, rank: int, placement: List[int], device=None) -> List[torch.nn.Module]:
    return get_handcrafted_imbalanced_partition(model, rank, placement, balanced_partition(len(model.blocks), placement), device)


def bench(model, parts, scheduler, placement, dtype=torch.float32, nmb: Optional[int] = None, ntrials: int = 1, stats_file: Optional[str] = None,
          n_iterations: int = 16, warmup: int = 3, optimizer_factory: Optional[Callable] = None, **pipeline_kwargs):
    """Time a pre-partitioned pipeline the way the reference's harness does
    (``benchmarks/benchmark_utils.py:69-143``): micro-batch size 1, ``nmb = 2 * world`` unless
    given, ``warmup`` untimed steps, then ``ntrials`` trials of ``n_iterations`` steps; returns
    ``(median seconds per iteration, peak GB of every rank (rank 0 only), all trial times)``.
    On GPUs a trial is timed with CUDA events and the maximum over ranks is taken; on CPU by
    wall clock.  ``optimizer_factory(params)`` adds an optimizer step to every iteration."""
    from elf_b200 import Pipeline, sequential_signatures

    world = dist.get_world_size() if dist.is_initialized() else 1
    rank = dist.get_rank() if dist.is_initialized() else 0
    n_micro_batches = nmb or 2 * world
    batch = n_micro_batches  # micro-batch size 1
    pipe = Pipeline(parts, None, placement=list(placement), partitioner=False, scheduler=scheduler, signatures=sequential_signatures(placement), **pipeline_kwargs)
    device = pipe.device
    on_cuda = device.type == "cuda"
    opt = optimizer_factory(list(pipe.parameters())) if optimizer_factory is not None else None

    def one_step():
        if opt is not None:
            opt.zero_grad()
        else:
            pipe.zero_grad(set_to_none=False)
        pipe(model.get_sample(batch, dtype, device), model.get_target(batch, dtype, device), model.loss_fn, split_size=1)
        if opt is not None:
            opt.step()

    for _ in range(warmup):
        one_step()
    if on_cuda:
        torch.cuda.reset_peak_memory_stats(device)
    times = []
    for _ in range(ntrials):
        if on_cuda:
            torch.cuda.synchronize(device)
        if world > 1:
            dist.barrier()
        t0 = time.perf_counter()
        if on_cuda:
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
        for _ in range(n_iterations):
            one_step()
        if on_cuda:
            b.record()
            torch.cuda.synchronize(device)
            secs = max_over_ranks(a.elapsed_time(b) / 1e3, device)
        else:
            if world > 1:
                dist.barrier()
            secs = time.perf_counter() - t0
        times.append(secs / n_iterations)
    peak = torch.cuda.max_memory_allocated(device) / 2**30 if on_cuda else 0.0
    peaks = None
    if world > 1:
        gathered = [None] * world if rank == 0 else None
        dist.gather_object(peak, gathered, dst=0)
        peaks = gathered
    elif rank == 0:
        peaks = [peak]
    if stats_file is not None:
        write_detailed_stats(stats_file, pipe.detailed_stats, rank, world)
    pipe.clear()
    return statistics.median(times), peaks, times


def check_correctness(model, pipe, atol: float = 1e-3, rtol: float = 1e-3, batch: Optional[int] = None) -> Dict[str, float]:
    """Compare one pipeline step with the same model run in a single process.

    The single-process copy is rebuilt on the rank that owns the last stage from
    ``pipe.gather_parameters`` (so it holds exactly the pipeline's weights), run on the same
    inputs, and outputs, loss and every parameter gradient are compared with
    ``atol`` / ``rtol`` (the reference's check, ``benchmarks/benchmark_utils.py:215-292``,
    uses 1e-3 for both).  ``model`` must be the un-partitioned module whose parameter names
    the stages kept (fx partitions do; hand-made ``nn.Sequential`` stages of ``model.blocks``
    do not).  The pipeline must have been built with ``outputs="cpu"`` or ``"device"``.
    Returns the largest absolute differences seen; raises ``AssertionError`` on a mismatch."""
    import copy

    world = dist.get_world_size() if dist.is_initialized() else 1
    rank = dist.get_rank() if dist.is_initialized() else 0
    device = pipe.device
    n = batch or 2 * max(1, pipe.pp)
    inputs = model.get_sample(n, device=device) if rank == 0 else None
    targets = model.get_target(n, device=device) if rank == 0 else None
    if world > 1:
        box = [inputs.cpu() if inputs is not None else None, targets.cpu() if targets is not None else None]
        dist.broadcast_object_list(box, src=0)
        inputs, targets = box[0].to(device), box[1].to(device)
    was_training = [b.model.training for b in pipe.blocks]
    for b in pipe.blocks:
        b.model.eval()  # no dropout on either side
    pipe.zero_grad()
    outputs, loss = pipe(inputs, targets, model.loss_fn, split_size=1)
    grads = {name: p.grad.detach().float().cpu() for name, p in pipe.named_parameters() if p.grad is not None}
    owner = (pipe.dp_rank * pipe.pp) + pipe.placement[-1]
    params = pipe.gather_parameters(dst=owner)
    report: Dict[str, float] = {}
    if world > 1:
        all_grads = [None] * world if rank == owner else None
        dist.gather_object(grads, all_grads, dst=owner)
    else:
        all_grads = [grads]
    if rank == owner:
        ref = copy.deepcopy(model)
        if any(p.is_meta for p in ref.parameters()):
            ref.to_empty(device="cpu")
        ref = ref.to("cpu").float()
        missing = ref.load_state_dict({k: v.detach().float().cpu() for k, v in params.items()}, strict=False)
        assert not missing.missing_keys, f"parameters the pipeline does not hold: {missing.missing_keys[:5]}"
        ref.eval()
        y_ref = ref(inputs.cpu())
        loss_ref = model.loss_fn(y_ref, targets.cpu())
        loss_ref.backward()
        for module in ref.modules():  # split-backward layers: run the deferred weight-gradient pass
            if hasattr(module, "move_last_computed") and hasattr(module, "backward") and hasattr(module, "ctx"):
                module.move_last_computed("input", 0)
                module.move_last_computed("grad_output", 0)
                module.backward(0)
        y = torch.cat([o.detach().float().cpu() for o in outputs]) if outputs else None
        if y is not None:
            report["output"] = float((y - y_ref.detach()).abs().max())
            torch.testing.assert_close(y, y_ref.detach(), atol=atol, rtol=rtol, msg=lambda m: f"pipeline output differs from the single-process model: {m}")
        report["loss"] = float((loss.detach().float().cpu() - loss_ref.detach()).abs())
        torch.testing.assert_close(loss.detach().float().cpu(), loss_ref.detach(), atol=atol, rtol=rtol, msg=lambda m: f"loss differs: {m}")
        ref_grads = {k: p.grad for k, p in ref.named_parameters() if p.grad is not None}
        worst = 0.0
        for part in all_grads:
            for name, g in part.items():
                assert name in ref_grads, f"gradient for {name} has no counterpart in the single-process model"
                worst = max(worst, float((g - ref_grads[name]).abs().max()))
                torch.testing.assert_close(g, ref_grads[name], atol=atol, rtol=rtol, msg=lambda m, name=name: f"gradient of {name} differs: {m}")
        report["grad"] = worst
    for b, t in zip(pipe.blocks, was_training):
        b.model.train(t)
    pipe.zero_grad()
    if world > 1:
        dist.barrier()
    return report
