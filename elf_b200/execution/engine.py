"""Schedule interpreter: runs this rank's slice of a schedule over its blocks.

Counterpart of the reference's ``Engine`` (``elf/execution/engine.py:96-371``) with the same
observable behaviour — the loss convention of ``compute_loss`` (``:374-410``), same-rank
hand-offs without p2p (``:413-445``), the ``stats`` / ``detailed_stats`` dictionaries and
the ``ELF_TIMINGS`` / ``ELF_MEMORY`` / ``ELF_PREALLOCATE_POOL`` switches — but:

* it runs on CPU tensors as well (no unconditional ``torch.cuda`` calls);
* dispatch is a table of bound handlers instead of a ``match`` per op;
* one ``OffloadManager`` (two side streams, one pinned arena) serves every
  (stage, micro-batch) instead of two fresh streams per offloader per step;
* outputs are copied to the host only when asked to (``outputs="cpu"``);
* gradient all-reduce handles are waited before the step returns.
"""

from __future__ import annotations

import contextlib
import logging
import os
import time
from collections import OrderedDict
from typing import Callable, Dict, List, Optional, Sequence

import torch
import torch.distributed as dist

from ..scheduling.scheduling import Operation, OperationType, OpOptions
from ..utils import stream_debug as _sd
from ..utils.timers import Timer
from .block import PipelineBlock
from .offload import OffloadManager, OffloadToCPU, PinnedHostTensorPool

logger = logging.getLogger("engine")

__all__ = ["Engine", "compute_loss", "preallocate_pool"]

T = OperationType
_COMPUTE_LIKE = (T.FORWARD, T.BACKWARD_INPUTS, T.BACKWARD_PARAMS, T.RECOMPUTE_FORWARD, T.RECOMPUTE_BACKWARD_INPUTS, T.LOSS_FORWARD, T.LOSS_BACKWARD)
_GIB = 1 << 30
_POOL_DTYPES = {
    "bf16": torch.bfloat16,
    "bfloat16": torch.bfloat16,
    "f16": torch.float16,
    "fp16": torch.float16,
    "float16": torch.float16,
    "f32": torch.float32,
    "fp32": torch.float32,
    "float32": torch.float32,
    "f64": torch.float64,
    "u8": torch.uint8,
}


def _env_flag(name: str) -> bool:
    return os.environ.get(name, "0").lower() not in ("", "0", "false", "no")


def preallocate_pool(pool: PinnedHostTensorPool, spec: Optional[str] = None) -> None:
    """Reserve pinned host memory up front from ``ELF_PREALLOCATE_POOL="bf16:8,f32:2"``
    (GiB per dtype), so the first offloading steps do not pay for ``cudaHostAlloc``."""
    spec = os.environ.get("ELF_PREALLOCATE_POOL", "") if spec is None else spec
    for item in filter(None, (s.strip() for s in spec.split(","))):
        try:
            name, gib = item.split(":")
            pool.reserve(int(float(gib) * _GIB), _POOL_DTYPES[name.strip().lower()])
        except (ValueError, KeyError):
            logger.warning("ELF_PREALLOCATE_POOL: cannot parse %r (expected e.g. 'bf16:8,f32:2')", item)


def compute_loss(block: PipelineBlock, output: torch.Tensor, target: torch.Tensor, loss_fn: Callable, grad_scale: float = 1.0):
    """Loss of one micro-batch and a closure that back-propagates it to ``output``.

    ``loss_fn`` is called with ``reduction="sum"`` (or without the keyword if it does not
    accept it) and the result is divided by the number of target elements per sample;
    the pipeline later divides by the batch size, which makes the step loss the mean over
    all elements of all samples.  ``grad_scale`` multiplies what is back-propagated (not the
    returned loss): with ``1 / batch size`` every gradient of the step comes out already
    scaled for the mean loss, and the separate pass over all gradients that the reference
    makes at the end of the step (``elf/execution/block.py:518-527``) is not needed."""
    leaf = output.detach().requires_grad_()
    timer = Timer(name="loss_forward")
    block.compute_time.append(timer)
    with timer:
        try:
            loss = loss_fn(leaf, target, reduction="sum")
        except TypeError:
            loss = loss_fn(leaf, target)
    per_sample = max(1, target.numel() // max(1, target.size(0))) if target.dim() else 1
    loss = loss / per_sample

    def grad_fn():
        (loss if grad_scale == 1.0 else loss * grad_scale).backward()
        return (leaf.grad.data,)

    return loss.detach(), grad_fn


class Engine:
    def __init__(self, blocks: Sequence[PipelineBlock], outputs: str = "cpu"):
        self.blocks = list(blocks)
        self.rank = self.blocks[0].rank if self.blocks else None
        for b in self.blocks:
            assert b.rank == self.rank, "All blocks in a stage should be on the same rank"
        self.id_to_block: Dict[int, PipelineBlock] = {b.id: b for b in self.blocks}
        self.device = self.blocks[0].device if self.blocks else torch.device("cpu")
        self.on_cuda = self.device.type == "cuda"
        self.outputs = outputs
        self.pool = PinnedHostTensorPool()
        preallocate_pool(self.pool)
        self.offload = OffloadManager(self.device, self.pool)
        self.result_stream = torch.cuda.Stream(self.device) if self.on_cuda else None
        self.last_step_events = None
        self._handlers = {
            T.FORWARD: self._forward,
            T.BACKWARD_INPUTS: self._backward_inputs,
            T.BACKWARD_PARAMS: self._backward_params,
            T.SEND_FORWARD: self._send_forward,
            T.SEND_BACKWARD: self._send_backward,
            T.RECV_FORWARD: self._recv_forward,
            T.RECV_BACKWARD: self._recv_backward,
            T.LOSS_FORWARD: self._loss_forward,
            T.LOSS_BACKWARD: self._loss_backward,
            T.RECOMPUTE_FORWARD: lambda b, op: b.recompute_forward(op.mb_id, **op.options),
            T.RECOMPUTE_BACKWARD_INPUTS: lambda b, op: b.recompute_backward_inputs(op.mb_id, **op.options),
            T.PREFETCH_ACTIVATIONS: lambda b, op: self._offloader(b.id, op.mb_id).prefetch(),
            # gradients are born scaled by 1 / batch size (see compute_loss): only the replica average is left
            T.ALL_REDUCE_PARAM_GRADS: lambda b, op: b.sync_grads(1),
        }

    # ------------------------------------------------------------------ op handlers
    def _offloader(self, block_id: int, mb: int) -> OffloadToCPU:
        key = (block_id, mb)
        off = self._offloaders.get(key)
        if off is None:
            off = self._offloaders[key] = self.offload.offloader(exclude=self.id_to_block[block_id].model.parameters())
        return off

    def _forward(self, block: PipelineBlock, op: Operation):
        ctx = self._offloader(block.id, op.mb_id) if op.options.get(OpOptions.ACTIVATION_OFFLOAD) else contextlib.nullcontext()
        with ctx:
            y = block.forward(op.mb_id, **op.options)
        if y is not None:
            self._results[op.mb_id] = [t.detach() if isinstance(t, torch.Tensor) else t for t in y]
            if self.on_cuda and _sd.enabled():
                for t in self._results[op.mb_id]:
                    if isinstance(t, torch.Tensor):
                        _sd.note_write(t, torch.cuda.current_stream(self.device), "output of the last stage")

    def _backward_inputs(self, block: PipelineBlock, op: Operation):
        block.backward_inputs(op.mb_id, **op.options)
        if op.options.get(OpOptions.ACTIVATION_OFFLOAD):
            self._offloader(block.id, op.mb_id).release()

    def _backward_params(self, block: PipelineBlock, op: Operation):
        block.backward_params(op.mb_id, **op.options)

    def _send_forward(self, block: PipelineBlock, op: Operation):
        dst = self.id_to_block.get(op.options.get("dst"))
        if dst is not None:  # same rank: move the tensors slot to slot, matched by order
            outs = [v for var_dsts in block.output_variables for v in var_dsts if v.peer_id == dst.id]
            ins = [v for v in dst.input_variables if v.peer_id == block.id]
            for src_var, dst_var in zip(outs, ins):
                dst_var.set(dst_var.to_process, op.mb_id, src_var.get(src_var.to_send, op.mb_id))
            return
        block.send_forward(op.mb_id, **op.options)

    def _send_backward(self, block: PipelineBlock, op: Operation):
        dst = self.id_to_block.get(op.options.get("dst"))
        if dst is not None:
            ins = [v for v in block.input_variables if v.peer_id == dst.id]
            outs = [v for var_dsts in dst.output_variables for v in var_dsts if v.peer_id == block.id]
            for src_var, dst_var in zip(ins, outs):
                if src_var.to_send.get(op.mb_id) is not None:
                    dst_var.set(dst_var.to_process, op.mb_id, src_var.get(src_var.to_send, op.mb_id))
            return
        block.send_backward(op.mb_id, **op.options)

    def _recv_forward(self, block: PipelineBlock, op: Operation):
        if block.is_first and op.options.get("src") is None:
            for tensor, var in zip(self._microbatches[op.mb_id], block.input_variables):
                var.set(var.to_process, op.mb_id, tensor)
            return
        block.recv_forward(op.mb_id, self._mb_sizes[op.mb_id], **op.options)

    def _recv_backward(self, block: PipelineBlock, op: Operation):
        block.recv_backward(op.mb_id, self._mb_sizes[op.mb_id], **op.options)

    def _loss_forward(self, block: PipelineBlock, op: Operation):
        if not block.is_last:
            logger.warning("Tried to compute loss on a non-last block %s", block)
            return
        assert op.mb_id in self._results, f"Loss forward for mb {op.mb_id} before its forward"
        assert self._targets is not None, "a target is required on the rank that owns the last stage"
        loss, grad_fn = compute_loss(block, self._results[op.mb_id][0], self._targets[op.mb_id], self._loss_fn, 1.0 / self._batch_size)
        self._losses[op.mb_id] = loss
        self._grad_fns[op.mb_id] = grad_fn

    def _loss_backward(self, block: PipelineBlock, op: Operation):
        if not block.is_last:
            logger.warning("Tried to compute loss backward on a non-last block %s", block)
            return
        grad_fn = self._grad_fns.pop(op.mb_id)
        timer = Timer(name=f"backward({block.id}:{op.mb_id})")
        block.compute_time.append(timer)
        with timer:
            grads = grad_fn()
        self._stash_result(op.mb_id)
        for grad, var_dsts in zip(grads, block.output_variables):
            for var in var_dsts:
                var.set(var.to_process, op.mb_id, grad)

    def _stash_result(self, mb: int) -> None:
        """Apply the ``outputs`` policy to the forward result of ``mb``."""
        if self.outputs in (None, False, "none"):
            self._results[mb] = None
        elif self.outputs == "cpu" and self.on_cuda:
            cur = torch.cuda.current_stream(self.device)
            self.result_stream.wait_stream(cur)
            _sd.note_sync(self.result_stream, cur)
            with torch.cuda.stream(self.result_stream), torch.no_grad():
                moved = []
                for t in self._results[mb]:
                    if isinstance(t, torch.Tensor):
                        _sd.check_read(t, self.result_stream, "copy of a result to the host")
                        t.record_stream(self.result_stream)
                        t = t.to("cpu", non_blocking=True)
                    moved.append(t)
                self._results[mb] = moved

    # ------------------------------------------------------------------ the step
    def train_step(self, batch, target, loss_fn, schedule: Sequence[Operation], mb_sizes: List[int], profile: bool = False):
        """Returns ``(result, losses, stats, detailed_stats)``.

        ``result``  per micro-batch outputs of the last stage (list; empty elsewhere)
        ``losses``  per micro-batch loss tensors
        ``stats``   ``total, idle, start_idle, end_idle, bubble`` in seconds; compute time
                    (hence idle/bubble) is measured only when ``ELF_TIMINGS`` is set
        ``detailed_stats``  ``all_events`` {timer name: s}, ``memories`` / ``peak_memory``
                    {str(op): bytes} (peaks are per-op only when ``ELF_MEMORY`` is set);
                    with ``ELF_TIMINGS`` also ``timeline`` {timer name: (begin s, end s)} on the
                    device clock, counted from the start of the step, and ``host_enqueue``
                    {str(op): s} = when the host issued the operation
        """
        precise_timings = _env_flag("ELF_TIMINGS")
        precise_memory = _env_flag("ELF_MEMORY")
        mb_sizes = list(mb_sizes)
        self._mb_sizes = mb_sizes
        self._batch_size = sum(mb_sizes)
        self._loss_fn = loss_fn
        self._microbatches = None
        if batch is not None:
            splits = [t.split(mb_sizes, dim=0) for t in batch]
            self._microbatches = list(zip(*splits))
        self._targets = target.split(mb_sizes, dim=0) if target is not None else None
        self._results: Dict[int, Optional[list]] = {}
        self._losses: Dict[int, torch.Tensor] = {}
        self._grad_fns: Dict[int, Callable] = {}
        self._offloaders: Dict[tuple, OffloadToCPU] = {}

        if precise_timings:
            if dist.is_initialized():
                dist.barrier()
            if self.on_cuda:
                torch.cuda.synchronize(self.device)
        if self.on_cuda:
            ev_start = torch.cuda.Event(enable_timing=True)
            ev_end = torch.cuda.Event(enable_timing=True)
            ev_start.record()
        pipe_start = time.perf_counter()
        warmup_time = None
        memories: "OrderedDict[str, int]" = OrderedDict()
        peaks: "OrderedDict[str, int]" = OrderedDict()
        host_enqueue: Dict[str, float] = {}  # when the host issued each compute operation (ELF_TIMINGS only)

        for op in schedule:
            block = self.id_to_block.get(op.block_id)
            if block is None:
                continue
            if profile and self.on_cuda:
                torch.cuda.nvtx.range_push(f"{block}:{op}")
            if precise_memory and self.on_cuda:
                torch.cuda.reset_peak_memory_stats(self.device)
            if warmup_time is None and op.op is not T.RECV_FORWARD:
                warmup_time = 0.0
                if precise_timings and not self.on_cuda:
                    warmup_time = time.perf_counter() - pipe_start
            handler = self._handlers.get(op.op)
            if handler is None:
                raise RuntimeError(f"Unknown operation : {op}")
            if precise_timings and op.op in _COMPUTE_LIKE:
                host_enqueue[str(op)] = time.perf_counter() - pipe_start
            handler(block, op)
            if self.on_cuda:
                if precise_memory:
                    torch.cuda.synchronize(self.device)
                memories[str(op)] = torch.cuda.memory_allocated(self.device)
                peaks[str(op)] = torch.cuda.max_memory_allocated(self.device)
            if profile and self.on_cuda:
                torch.cuda.nvtx.range_pop()

        for block in self.blocks:
            block.wait_grad_sync()
        if self.on_cuda:
            ev_end.record()
            self.last_step_events = (ev_start, ev_end)
        cooldown_start = time.perf_counter()
        if precise_timings and self.on_cuda:
            torch.cuda.synchronize(self.device)
        pipe_end = time.perf_counter()

        compute_time = 0.0
        all_events: Dict[str, float] = {}
        timeline: Dict[str, tuple] = {}
        if precise_timings:
            for block in self.blocks:
                for timer in block.compute_time:
                    t = timer.time()
                    compute_time += t
                    all_events[timer.name] = t
                    key, k = timer.name, 0
                    while key in timeline:  # timers that share a name (loss_forward): keep them all
                        k += 1
                        key = f"{timer.name}#{k}"
                    if self.on_cuda and hasattr(timer, "start_event"):
                        # begin / end of the operation on the device, seconds after the step's start event
                        t0 = ev_start.elapsed_time(timer.start_event) / 1e3
                        timeline[key] = (t0, t0 + t)
                    elif hasattr(timer, "start"):
                        timeline[key] = (timer.start - pipe_start, timer.end - pipe_start)
        if precise_timings and self.on_cuda and timeline:
            # time until the first operation starts on the device, read from the events: a device
            # synchronisation here would also wait for receives posted ahead of their use
            warmup_time = max(0.0, min(t0 for t0, _ in timeline.values()))
        total = pipe_end - pipe_start
        stats = {
            "total": total,
            "idle": total - compute_time,
            "start_idle": warmup_time or 0.0,
            "end_idle": pipe_end - cooldown_start,
        }
        stats["bubble"] = stats["idle"] - stats["start_idle"] - stats["end_idle"]
        detailed = {"all_events": all_events, "memories": memories, "peak_memory": peaks, "timeline": timeline, "host_enqueue": host_enqueue}
        for block in self.blocks:
            block.compute_time.clear()

        if self.on_cuda:
            torch.cuda.current_stream(self.device).wait_stream(self.result_stream)
        self.offload.finish_step(self._offloaders.values())
        self._offloaders = {}

        result = []
        for mb in sorted(self._results):
            r = self._results[mb]
            if r is not None:
                result.append(r[0] if len(r) == 1 else r)
        losses = [self._losses[mb] for mb in sorted(self._losses)]
        self._results, self._grad_fns, self._microbatches, self._targets = {}, {}, None, None
        return result, losses, stats, detailed

    def device_step_ms(self) -> Optional[float]:
        """Device time of the last step (CUDA events around the schedule loop); blocks."""
        if not self.last_step_events:
            return None
        a, b = self.last_step_events
        b.synchronize()
        return a.elapsed_time(b)
