"""``Pipeline``: the user-facing object that partitions a model over pipeline ranks, builds
the runtime and runs training steps.

API and behaviour follow the reference (``elf/pipeline.py``): ``Pipeline(model, sample,
placement=, partitioner=, scheduler=, comm_scheduler=, tracer=, pp=, dp=, worker=,
memory_budget=, signatures=)``, ``pipe(batch, target, loss_fn, split_size=, profile=,
scheduler=)``, ``parameters/named_parameters``, ``zero_grad``, ``clear``,
``checkpoint``, ``save``, ``gather_parameters``, ``is_first/is_last``,
``get_profiling_statistics``, attributes ``stats``, ``detailed_stats``, ``blocks``,
``engine``, ``placement``, ``signatures``, ``schedule``, ``pp``, ``dp``, ``dp_rank``.

Deliberate differences:

* placements and schedules use pipeline-local ranks ``0..pp-1`` on every data-parallel
  replica; the replica offset is applied only when addressing ``torch.distributed`` peers,
  so every scheduler works with ``dp > 1`` (the reference shifts the placement itself,
  ``elf/pipeline.py:165-168``);
* runs without ``torch.distributed`` (single process = one stage chain on one device) and
  on CPU/gloo;
* ``load_checkpoint`` restores what ``checkpoint`` wrote; ``save`` works for every rank;
* ``scheduler="auto"`` without a memory budget means 1F1B instead of failing later;
* extra options: ``outputs`` ("cpu" as the reference, "device", or "none"),
  ``grad_sync`` ("auto" | "nccl" | "symm"), ``offload`` (the ILP may offload activations) and
  ``p2p`` ("auto" | "nccl" | "copy": transport between stages).
"""

from __future__ import annotations

import logging
import os
from dataclasses import dataclass, field, fields
from datetime import timedelta
from typing import Any, Callable, Dict, Iterator, List, Optional, Tuple, Union

import torch
import torch.distributed as dist
import torch.nn as nn

from .execution.block import PipelineBlock
from .execution.channels import ChannelTable
from .execution.engine import Engine
from .partitioners.signature import Signature, sequential_signatures
from .registry import COMM_SCHEDULERS, PARTITIONERS, SCHEDULERS, TRACERS, resolve
from .scheduling import add_comms, check_schedule_validity, schedule_to_str
from .scheduling.scheduling import OperationType
from .utils.placement import Placement
from .utils.shipping import broadcast_models, recv_models, send_models, transport_device

logger = logging.getLogger("pipeline")

__all__ = ["Pipeline", "PipelineConfig"]


@dataclass
class PipelineConfig:
    """Options of a ``Pipeline``.

    tracer          key of ``TRACERS`` or callable ``(model, sample) -> fx.GraphModule``
    partitioner     key of ``PARTITIONERS``, callable, or ``False`` for a pre-partitioned model
    scheduler       key of ``SCHEDULERS`` or callable ``(placement, nmb) -> List[Operation]``
    comm_scheduler  key of ``COMM_SCHEDULERS``, callable, or ``False``
    placement       ``"auto"`` (from the scheduler) or a list stage → pipeline rank
    pp, dp          pipeline / data parallel sizes (``pp`` defaults to ``world // dp``)
    worker          rank that traces, partitions and solves the ILP
    memory_budget   per-GPU budget in **MB**; enables ILP rematerialisation
    offload         with a memory budget: let the ILP also park activations in pinned host memory
    signatures      stage signatures of a pre-partitioned model
    """

    tracer: Union[str, Callable] = field(default="default", metadata={"registry": TRACERS})
    partitioner: Union[str, Callable, bool] = field(default="constrained", metadata={"registry": PARTITIONERS})
    scheduler: Union[str, Callable] = field(default="auto", metadata={"registry": SCHEDULERS})
    comm_scheduler: Union[str, Callable, bool] = field(default="pipelined", metadata={"registry": COMM_SCHEDULERS})
    placement: Union[str, List[int]] = "auto"
    pp: Optional[int] = None
    dp: int = 1
    worker: int = 0
    memory_budget: Optional[float] = None
    signatures: Optional[List[Signature]] = None
    outputs: str = "cpu"
    grad_sync: str = "auto"
    offload: bool = False
    p2p: str = "auto"

    def resolve(self) -> "PipelineConfig":
        """Copy with registry keys replaced by the registered callables (``False`` stays)."""
        values = {}
        for f in fields(self):
            v = getattr(self, f.name)
            reg = f.metadata.get("registry")
            if reg is not None and v is not False and v is not None:
                v = resolve(v, reg)
            values[f.name] = v
        return PipelineConfig(**values)

    def to_kwargs(self) -> dict:
        return {f.name: getattr(self, f.name) for f in fields(self) if getattr(self, f.name) is not None}


def _world() -> Tuple[int, int]:
    if dist.is_available() and dist.is_initialized():
        return dist.get_rank(), dist.get_world_size()
    return 0, 1


class Pipeline:
    def __init__(self, model, sample=None, *, config: Optional[PipelineConfig] = None, **kwargs):
        rank, ws = _world()
        if ws == 1 and not (dist.is_available() and dist.is_initialized()):
            logger.info("torch.distributed is not initialised: running the whole pipeline in this process")
        self.rank, self.world_size = rank, ws
        raw = config or PipelineConfig(**kwargs)
        self._scheduler_name = raw.scheduler if isinstance(raw.scheduler, str) else None
        if raw.scheduler == "auto" and raw.memory_budget is None:
            logger.info("scheduler='auto' without memory_budget: using 1f1b")
            raw = PipelineConfig(**{**raw.to_kwargs(), "scheduler": "1f1b"})
            self._scheduler_name = "1f1b"
        self.cfg = raw.resolve()

        self.dp = int(self.cfg.dp)
        self.pp = int(self.cfg.pp or ws // self.dp)
        assert self.pp * self.dp == ws, f"Requested PP = {self.pp}, DP = {self.dp} need {self.pp * self.dp} processes, but {ws} were spawned"
        self.dp_rank = rank // self.pp
        self.pp_rank = rank % self.pp

        if isinstance(self.cfg.placement, str) and self.cfg.placement == "auto":
            name = self._scheduler_name
            if name is None:
                try:
                    name = SCHEDULERS.get_key(self.cfg.scheduler)
                except ValueError:
                    name = ""
            self.placement = Placement.default(name, self.pp)
        else:
            self.placement = Placement(self.cfg.placement).normalised()
        assert max(self.placement) < self.pp, f"placement {list(self.placement)} uses more than pp={self.pp} ranks"

        self.device = transport_device() if (dist.is_available() and dist.is_initialized()) else (
            torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else torch.device("cpu")
        )
        self._init_process_groups()

        self.scheduler = self.cfg.scheduler
        self.tracer = self.cfg.tracer
        self.partitioner = self.cfg.partitioner

        parts, signatures = self._partition_model(model, sample, self.cfg.signatures)
        self.signatures = signatures
        self.blocks = self._create_pipeline(parts, signatures)
        self.engine = Engine(self.blocks, outputs=self.cfg.outputs)
        self._configure_grad_sync()

        self._transport_decided = False
        self.schedule: list = []
        self.full_schedule: list = []
        self.last_nmb = 0
        self.stats: dict = {}
        self.detailed_stats: dict = {}

        self._remat_stats = None
        if self.cfg.memory_budget is not None:
            from .scheduling.ilp import AutoScheduler, profile_all_stages, stagerematify

            assert sample is not None, "sample is required when memory_budget is set (used for profiling)"
            self._remat_stats = profile_all_stages(self.blocks, self.signatures, self.placement, sample, self.pp_group)
            if self._scheduler_name == "auto":
                self.scheduler = AutoScheduler(self._remat_stats, self.cfg.memory_budget, self.cfg.worker, group=self.pp_group, offload=bool(self.cfg.offload))
            else:
                self.scheduler = stagerematify(self.scheduler, self._remat_stats, self.cfg.memory_budget, self.cfg.worker, group=self.pp_group, offload=bool(self.cfg.offload))

    # ------------------------------------------------------------------ set-up
    def _to_global(self, pp_local_rank: int) -> int:
        return self.dp_rank * self.pp + pp_local_rank

    def _init_process_groups(self) -> None:
        """One PP group per replica, one DP group per pipeline position; optional
        ``ELF_TIMEOUT`` seconds as group timeout."""
        self.pp_group = None
        self.dp_groups: List[Any] = []
        self._timeout = None
        if self.world_size == 1:
            return
        t = os.getenv("ELF_TIMEOUT")
        self._timeout = timedelta(seconds=int(t)) if t else None
        kw = {"timeout": self._timeout} if self._timeout is not None else {}
        if self.dp == 1:
            self.pp_group = dist.group.WORLD
            return
        for replica in range(self.dp):
            g = dist.new_group([replica * self.pp + r for r in range(self.pp)], **kw)
            if replica == self.dp_rank:
                self.pp_group = g
        for pos in range(self.pp):
            self.dp_groups.append(dist.new_group([d * self.pp + pos for d in range(self.dp)], **kw))

    def _partition_model(self, model, sample, signatures):
        local_ids = self.placement.get_ids(self.pp_rank)
        if not self.partitioner:
            parts = [model] if isinstance(model, nn.Module) else list(model)
            assert len(parts) == len(local_ids), f"rank {self.rank} hosts stages {local_ids} but got {len(parts)} module(s)"
            if signatures is None:
                if self.rank == 0:
                    logger.warning("No signatures provided, assuming sequential partitioning.")
                signatures = sequential_signatures(self.placement)
            return parts, signatures
        assert sample is not None, "Sample is required for partitioning"
        try:
            return self._shared_partition(model, sample)
        except Exception:
            logger.error("Error partitioning the model: it may use features that torch.fx/torch.export or this library do not support.")
            raise

    def _shared_partition(self, model, sample):
        """The worker rank traces, profiles and cuts the model, keeps its own stages and
        ships the others (skeleton by pickle, tensors in bulk); replicas get theirs by
        broadcast over the DP group of their pipeline position."""
        from .partitioners import partition

        n_local = self.placement.count(self.pp_rank)
        blocks: List[Any] = [None] * n_local
        signatures: List[Any] = [None] * len(self.placement)
        worker = self.cfg.worker
        if self.rank == worker:
            result = partition(model, len(self.placement), sample, partitioner=self.partitioner, tracer=self.tracer)
            parts = result.create_blocks()
            signatures = result.signatures
            self.partition_result = result
            for d in range(self.pp):
                on_d = [parts[i] for i in range(len(parts)) if self.placement[i] == d]
                if d == self.pp_rank:
                    blocks = on_d
                elif self.world_size > 1:
                    send_models(on_d, dst=self._to_global(d), group=self.pp_group)
                    dist.send_object_list(signatures, dst=self._to_global(d), group=self.pp_group)
        elif self.dp_rank == worker // self.pp:
            recv_models(blocks, src=worker, group=self.pp_group, device=self.device)
            dist.recv_object_list(signatures, src=worker, group=self.pp_group)
        if self.dp > 1:
            src = (worker // self.pp) * self.pp + self.pp_rank
            broadcast_models(blocks, src=src, group=self.dp_groups[self.pp_rank], device=self.device)
            dist.broadcast_object_list(signatures, src=src, group=self.dp_groups[self.pp_rank])
        return blocks, signatures

    def _create_pipeline(self, parts, signatures) -> List[PipelineBlock]:
        ids = self.placement.get_ids(self.pp_rank)
        self.channels = None
        if self.world_size > 1:
            self.channels = ChannelTable(
                self.placement, signatures, self.pp_rank, self.pp_group, self.device,
                pp=self.pp, dp=self.dp, dp_rank=self.dp_rank, timeout=self._timeout,
            )
        blocks = []
        for part, block_id in zip(parts, ids):
            dp_group = self.dp_groups[self.pp_rank] if self.dp > 1 else None
            blocks.append(
                PipelineBlock(part, block_id, self.placement, signatures[block_id], pp_group=self.pp_group, dp_group=dp_group,
                              channels=self.channels, device=self.device, rank=self.pp_rank)
            )
        if self.world_size > 1:
            dist.barrier(self.pp_group)
        return blocks

    def _configure_grad_sync(self) -> None:
        """Pick the data-parallel gradient path: the symmetric-memory push kernels on CUDA
        (``elf_b200.parallel.dp_sync``) or plain all-reduce."""
        mode = self.cfg.grad_sync
        self.grad_sync = None
        if self.dp == 1 or mode == "nccl" or self.device.type != "cuda":
            return
        try:
            from .parallel.dp_sync import SymmetricGradSync

            self.grad_sync = SymmetricGradSync(self.blocks, self.dp_groups[self.pp_rank])
            for b in self.blocks:
                b._grad_sync = self.grad_sync
        except Exception as exc:
            if mode == "symm":
                raise
            logger.warning("symmetric-memory gradient sync unavailable (%s); using all-reduce", exc)

    # ------------------------------------------------------------------ the step
    def step(self, batch, target, loss_fn, split_size=0, profile=False, scheduler=None):
        """Run one training (or inference) step.

        Returns ``(outputs, loss)`` on the rank hosting the last stage — ``outputs`` is a
        list with one entry per micro-batch (on the host unless ``outputs="device"``;
        empty for ``outputs="none"``), ``loss`` the mean loss over the batch, averaged over
        replicas — and ``(None, None)`` elsewhere.  Gradients are left in ``p.grad``,
        scaled for the mean loss and averaged over replicas; they accumulate across calls
        until ``zero_grad``."""
        if self.device.type == "cuda":
            from .ops import gemm as _gemm

            _gemm.raise_if_failed(self.device)  # a bounded device wait that ran out in an earlier step
        if batch is not None and isinstance(batch, torch.Tensor):
            batch = [batch]
        mb_sizes = self._get_mb_sizes(split_size, batch)
        nmb = len(mb_sizes)
        regenerate = scheduler is not None or nmb != self.last_nmb
        sched = self.scheduler if scheduler is None else resolve(scheduler, SCHEDULERS)
        if regenerate:
            self._generate_schedule(nmb, sched, self.cfg.comm_scheduler, mb_sizes)
            self.last_nmb = nmb if scheduler is None else 0
        PipelineBlock._step_counter += 1
        for block in self.blocks:
            for layer in block.dw_layers():
                layer.clear()
        if self.grad_sync is not None and any(op.op is OperationType.ALL_REDUCE_PARAM_GRADS for op in self.schedule):
            # only a step that exchanges gradients opens a new exchange epoch (and flips the inbox
            # parity): an inference step in between must not let the next training step write
            # into the half of the inbox a slower replica may still be reading
            self.grad_sync.begin_step()

        if batch is not None:
            batch = [t.to(self.device, non_blocking=True) if t.device != self.device else t for t in batch]
        if target is not None and target.device != self.device:
            target = target.to(self.device, non_blocking=True)
        try:
            result, losses, stats, detailed = self.engine.train_step(batch, target, loss_fn, self.schedule, mb_sizes, profile)
        except BaseException:
            # an operation raised (user loss function, a peer that went away, ...): drop every
            # half-finished micro-batch so that the pipeline object stays usable - a later step,
            # ``clear()`` and checkpointing must not trip over stale slots or pending receives
            self._abandon_step()
            raise

        for block in self.blocks:
            block._wait_for_send_ops()
            block.clear_slots()
        if self.channels is not None:
            for ch in self.channels.channels.values():
                ch.end_step()
            self._maybe_switch_transport()
        self.stats, self.detailed_stats = stats, detailed
        if self.device.type == "cuda":
            _gemm.snapshot_status_async(self.device)

        if self.blocks and self.blocks[-1].is_last and (losses or result):
            loss = None
            if losses:
                with torch.no_grad():
                    loss = torch.stack([l.detach().float().reshape(()) for l in losses]).sum() / sum(mb_sizes)
                if self.dp > 1:
                    g = self.blocks[-1].dp_group
                    if dist.get_backend(g) == "nccl":
                        dist.all_reduce(loss, group=g, op=dist.ReduceOp.AVG)
                    else:
                        dist.all_reduce(loss, group=g, op=dist.ReduceOp.SUM)
                        loss /= self.dp
            return result, loss
        return None, None

    __call__ = step

    def _maybe_switch_transport(self) -> None:
        """After the first completed step (which told every channel its message size over NCCL),
        move stage-to-stage traffic to the copy-engine transport: with ``p2p="copy"``, and with
        ``"auto"`` whenever the tensors are on CUDA devices and the groups are NCCL (the
        ``ELF_B200_P2P`` environment variable overrides ``"auto"``).  Measured on two B200s with
        the Llama-3-8B shape: 1561 ms per step against 1622 ms over NCCL send/recv."""
        if self._transport_decided:
            return
        self._transport_decided = True
        auto = self.cfg.p2p == "auto" and "ELF_B200_P2P" not in os.environ
        want = self.cfg.p2p if self.cfg.p2p != "auto" else os.environ.get("ELF_B200_P2P", "copy")
        if want != "copy":
            return
        if self.device.type != "cuda" or self.channels.transport != "nccl":
            if not auto:
                logger.warning("p2p='copy' needs CUDA devices and NCCL process groups; staying on %s", self.channels.transport)
            return
        timeout_ms = 1e3 * self._timeout.total_seconds() if self._timeout is not None else 60000.0
        n = self.channels.upgrade_to_copy(timeout_ms=timeout_ms)
        logger.info("rank %d: %d channel(s) now use the copy-engine transport", self.rank, n)

    def _abandon_step(self) -> None:
        """Forget the state of a step that did not finish: slots, W-pass stashes, offloaded
        activations, posted receives and send handles (without waiting for peers)."""
        for block in self.blocks:
            try:
                block.clear_slots()
                block.compute_time.clear()
                block._pending_reduce.clear()
            except Exception:  # pragma: no cover - best effort while another error propagates
                logger.exception("while abandoning a step on %s", block)
        if self.channels is not None:
            for ch in self.channels.channels.values():
                ch.abandon()
        eng = self.engine
        try:
            eng.offload.finish_step(getattr(eng, "_offloaders", {}).values())
        except Exception:  # pragma: no cover
            logger.exception("while releasing offloaded activations")
        eng._offloaders = {}
        eng._results, eng._grad_fns, eng._losses = {}, {}, {}
        eng._microbatches = eng._targets = None

    def _get_mb_sizes(self, split_size, batch) -> List[int]:
        """``0`` → ``batch // pp`` per micro-batch; an int → equal chunks plus a remainder;
        a list → as given (must cover the batch)."""
        if batch is None:
            raise ValueError("every rank must pass a batch (only its size is used away from the first stage)")
        batch_size = batch[0].size(0)
        if isinstance(split_size, int):
            if split_size > batch_size:
                logger.warning("Split size %d is greater than batch size %d", split_size, batch_size)
                split_size = batch_size
            if split_size == 0:
                split_size = batch_size // self.pp if self.pp <= batch_size else 1
            sizes = [split_size] * (batch_size // split_size)
            if batch_size % split_size:
                sizes.append(batch_size % split_size)
            return sizes
        assert sum(split_size) == batch_size, "Splits do not cover the entire batch"
        return list(split_size)

    def _generate_schedule(self, n_micro_batches, scheduler, comm_scheduler, mb_sizes) -> None:
        schedule = scheduler(self.placement, n_micro_batches)
        schedule = add_comms(schedule, self.signatures)
        if comm_scheduler:
            schedule = comm_scheduler(schedule)
        check_schedule_validity(schedule)
        if self.rank == 0 and logger.isEnabledFor(logging.DEBUG):
            logger.debug("Schedule:\n%s", schedule_to_str(schedule))
        self.full_schedule = schedule
        mine = {b.id for b in self.blocks}
        self.schedule = [op for op in schedule if op.block_id in mine and op.rank == self.pp_rank]
        for block in self.blocks:  # the micro-batch whose W pass completes the stage's gradients
            ws = [op.mb_id for op in self.schedule if op.block_id == block.id and op.op.name == "BACKWARD_PARAMS"]
            block.final_w_mb = ws[-1] if ws else None

    # ------------------------------------------------------------------ parameters
    def parameters(self) -> Iterator[nn.Parameter]:
        for block in self.blocks:
            yield from block.model.parameters()

    def named_parameters(self) -> Iterator[Tuple[str, nn.Parameter]]:
        for block in self.blocks:
            yield from block.model.named_parameters()

    def zero_grad(self, set_to_none: bool = True) -> None:
        for block in self.blocks:
            block.model.zero_grad(set_to_none=set_to_none)

    def is_first(self) -> bool:
        return self.placement.is_head(self.pp_rank)

    def is_last(self) -> bool:
        return self.placement.is_tail(self.pp_rank)

    def set_scheduler(self, scheduler) -> None:
        """Replace the scheduler (a registry key or a callable ``(placement, nmb) -> schedule``);
        the schedule is regenerated on the next step."""
        self.scheduler = resolve(scheduler, SCHEDULERS)
        self.last_nmb = None

    def measured_stage_costs(self):
        """Mean measured duration, in seconds, of the forward, backward-inputs and backward-params
        operations of every stage of the pipeline during the last step, as a list of
        ``(f, b, w)`` triples indexed by stage — the same on every rank of the pipeline.

        The last step must have run with per-operation timers (``ELF_TIMINGS=1``).  Meant for
        profile-guided schedules: feed the list to a cost-aware scheduler such as
        ``functools.partial(generate_zbv_schedule, cap="auto", stage_costs=costs)`` and install
        it with ``set_scheduler``.  Stages without split backward report ``w = 0``; the last stage's
        ``b`` includes the loss and its backward."""
        import re

        events = (self.detailed_stats or {}).get("all_events") or {}
        if not events:
            raise RuntimeError("no per-operation timings: run a step with ELF_TIMINGS=1 first")
        acc: Dict[int, Dict[str, List[float]]] = {}
        for name, secs in events.items():
            m = re.match(r"(forward|backward_inputs|backward_params)\((\d+):\d+\)$", name)
            if m:
                acc.setdefault(int(m.group(2)), {}).setdefault(m.group(1), []).append(float(secs))
        # the loss and its backward run as operations of their own on the rank of the last stage:
        # they count towards that stage's backward, or the rank looks lighter than it is
        last = len(self.placement) - 1
        timeline = (self.detailed_stats or {}).get("timeline") or {}
        loss_f = [t1 - t0 for name, (t0, t1) in timeline.items() if name.split("#")[0] == "loss_forward"]
        loss_b = [float(secs) for name, secs in events.items() if re.match(rf"backward\({last}:\d+\)$", name)]
        loss_extra = (sum(loss_f) / len(loss_f) if loss_f else 0.0) + (sum(loss_b) / len(loss_b) if loss_b else 0.0)
        mine = {}
        for stage, kinds in acc.items():
            mean = lambda k: (sum(kinds[k]) / len(kinds[k])) if kinds.get(k) else 0.0
            mine[stage] = (mean("forward"), mean("backward_inputs") + (loss_extra if stage == last else 0.0), mean("backward_params"))
        parts = [mine]
        if self.pp_group is not None and dist.is_initialized() and dist.get_world_size(self.pp_group) > 1:
            parts = [None] * dist.get_world_size(self.pp_group)
            dist.all_gather_object(parts, mine, group=self.pp_group)
        merged: Dict[int, tuple] = {}
        for part in parts:
            merged.update(part)
        n_stages = len(self.placement)
        missing = [s for s in range(n_stages) if s not in merged]
        if missing:
            raise RuntimeError(f"no timings for stages {missing}")
        return [merged[s] for s in range(n_stages)]

    def get_profiling_statistics(self):
        if not self._remat_stats:
            raise ValueError("Profiling statistics are only available when the pipeline was built with a memory budget")
        return self._remat_stats

    # ------------------------------------------------------------------ teardown
    def clear(self) -> None:
        """Synchronise, then destroy the groups this pipeline created."""
        if self.device.type == "cuda":
            torch.cuda.synchronize(self.device)
        if self.world_size == 1:
            return
        dist.barrier()
        if self.grad_sync is not None:
            self.grad_sync.close()
        if self.channels is not None:
            self.channels.destroy()
        for g in self.dp_groups:
            try:
                dist.destroy_process_group(g)
            except Exception:
                pass
        if self.dp > 1 and self.pp_group is not None:
            dist.destroy_process_group(self.pp_group)
        self.dp_groups = []

    # ------------------------------------------------------------------ checkpoints
    def _ckpt_path(self, epoch, dir_path) -> str:
        return os.path.join(str(dir_path), str(epoch), f"dp{self.dp_rank}_pp{self.pp_rank}.pt")

    def checkpoint(self, epoch="init", dir_path="./", extra: Optional[dict] = None) -> str:
        """Write ``{dir_path}/{epoch}/dp{dp}_pp{pp}.pt`` with the reference's layout:
        ``rank, pp, dp, epoch`` and one ``state_dict_{block id}`` per local stage
        (``elf/pipeline.py:346-368``).  ``extra`` entries (optimizer state, step counters)
        are stored under their own keys, which older readers ignore."""
        state = {"rank": self.rank, "pp": self.pp_rank, "dp": self.dp_rank, "epoch": epoch}
        for block in self.blocks:
            state[f"state_dict_{block.id}"] = {k: v.data for k, v in block.model.state_dict().items()}
        if extra:
            state.update(extra)
        path = self._ckpt_path(epoch, dir_path)
        os.makedirs(os.path.dirname(path), exist_ok=True)
        torch.save(state, path)
        return path

    def load_checkpoint(self, epoch="init", dir_path="./", strict: bool = True) -> dict:
        """Restore this rank's stages from a ``checkpoint`` file; returns the whole
        dictionary so callers can pick up their ``extra`` entries."""
        path = self._ckpt_path(epoch, dir_path)
        if not os.path.isfile(path):
            raise FileNotFoundError(f"no checkpoint for dp={self.dp_rank}, pp={self.pp_rank} at {path}")
        try:
            state = torch.load(path, map_location=self.device, weights_only=False)
        except Exception as exc:
            raise RuntimeError(f"checkpoint {path} cannot be read (truncated or corrupt file?): {type(exc).__name__}: {exc}") from exc
        if not isinstance(state, dict):
            raise RuntimeError(f"checkpoint {path} does not hold a checkpoint dictionary (got {type(state).__name__})")
        held = sorted(int(k[len("state_dict_"):]) for k in state if isinstance(k, str) and k.startswith("state_dict_") and k[len("state_dict_"):].isdigit())
        for block in self.blocks:
            key = f"state_dict_{block.id}"
            if key not in state:
                raise RuntimeError(
                    f"checkpoint {path} has no entry for stage {block.id}: it holds stages {held} "
                    f"(written by pp rank {state.get('pp')}, dp rank {state.get('dp')}); was it saved with another placement?"
                )
        for block in self.blocks:
            try:
                block.model.load_state_dict(state[f"state_dict_{block.id}"], strict=strict)
            except RuntimeError as exc:
                raise RuntimeError(f"checkpoint {path}: stage {block.id} does not match this pipeline's stage: {exc}") from exc
        # optimizers with fp32 master weights over these parameters must follow the load, or
        # their next step would write the old weights back
        seen = set()
        for p in self.parameters():
            group = getattr(p, "_elf_flat_group", None)
            if group is None or id(group) in seen:
                continue
            seen.add(id(group))
            for ref in getattr(group, "optimizers", []):
                opt = ref()
                if opt is not None:
                    opt.resync_master()
        return state

    def gather_parameters(self, dst: int = 0) -> dict:
        """Merged ``{name: tensor}`` of all stages of this replica on global rank ``dst``
        (``{}`` elsewhere).  Names are the stage modules' own (for fx partitions these are
        the original model's qualified names)."""
        local = {}
        for block in self.blocks:
            for name, p in block.model.named_parameters():
                if name in local:
                    logger.warning("Duplicate parameter %s in block %s, keeping the first", name, block.id)
                else:
                    local[name] = p.data
        if self.world_size == 1:
            return dict(local)
        members = dist.get_process_group_ranks(self.pp_group)
        if dst not in members:
            return {}
        meta = {n: (tuple(t.shape), t.dtype) for n, t in local.items()}
        gathered = [None] * len(members) if self.rank == dst else None
        dist.gather_object(meta, gathered, dst=dst, group=self.pp_group)
        if self.rank == dst:
            out = dict(local)
            for peer, peer_meta in zip(members, gathered):
                if peer == dst:
                    continue
                for name, (shape, dtype) in peer_meta.items():
                    buf = torch.empty(shape, dtype=dtype, device=self.device)
                    dist.recv(buf, src=peer, group=self.pp_group)
                    out.setdefault(name, buf)
            return out
        for t in local.values():
            dist.send(t.contiguous().to(self.device), dst=dst, group=self.pp_group)
        return {}

    def save(self, path, worker: int = 0) -> None:
        """Gather every stage's parameters on ``worker`` and write one flat
        ``{name: cpu tensor}`` file."""
        state = self.gather_parameters(dst=worker)
        if self.rank == worker:
            torch.save({k: v.detach().cpu() for k, v in state.items()}, path)
            logger.info("Saved model to %s", path)
