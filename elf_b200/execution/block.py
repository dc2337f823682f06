"""One pipeline stage on one rank: slots for in-flight tensors and the op vocabulary.

``PipelineBlock`` implements every operation type of the schedule IR (forward,
backward-inputs, backward-params, recomputes, send/recv, gradient all-reduce) for one
stage module; ``Variable`` holds the per-micro-batch tensors travelling through one input
or one (output, destination) pair.  Semantics follow the reference
(``elf/execution/block.py``): slots are written once and read once, stage inputs are
detached leaves that require grad when floating, the outputs of a multi-consumer tensor
receive the sum of their consumers' gradients, and ``LayerDW`` layers get their W-pass
operands filed per micro-batch after F and B.

The block is device-agnostic (CPU tensors with gloo, CUDA tensors with NCCL) and talks to
its peers through ``Channel`` objects (``elf_b200/execution/channels.py``).
"""

from __future__ import annotations

import logging
from typing import Dict, List, Optional

import torch
import torch.distributed as dist

from ..scheduling.scheduling import OpOptions
from ..utils.metadata import TensorMetadata
from ..utils.timers import Timer
from ..zb_utils import LayerDW, partial_dx_recomputation
from .remat import RematManager

logger = logging.getLogger("block")

__all__ = ["Variable", "PipelineBlock"]


class _Slots(dict):
    """Per-micro-batch single-assignment storage."""

    def put(self, mb: int, value) -> None:
        if self.get(mb) is not None:
            raise ValueError(f"slot {mb} already holds a value")
        self[mb] = value

    def take(self, mb: int, delete: bool = True):
        if self.get(mb) is None:
            raise KeyError(f"slot {mb} is empty")
        return self.pop(mb) if delete else self[mb]


class Variable:
    """A named tensor crossing a stage boundary, seen from one block.

    ``to_process``  what arrived (or will arrive) from ``peer_id`` and awaits compute
    ``saved``       what the block keeps between its F and its B
    ``to_send``     what the block produced for ``peer_id``
    """

    def __init__(self, name: str, peer_id: Optional[int], group=None):
        self.name = name
        self.peer_id = peer_id
        self.group = group
        self.to_process = _Slots()
        self.saved = _Slots()
        self.to_send = _Slots()
        self.metadata: Optional[TensorMetadata] = None
        self.was_metadata_sent = False
        self.recv_channel = None  # Channel delivering to_process entries, if remote

    def set(self, queue: _Slots, mb_id: int, value) -> None:
        try:
            queue.put(mb_id, value)
        except ValueError as exc:
            raise ValueError(f"{self}: {exc}") from None

    def get(self, queue: _Slots, mb_id: int, delete: bool = True):
        try:
            return queue.take(mb_id, delete)
        except KeyError as exc:
            raise KeyError(f"{self}: {exc}") from None

    def wait_and_pop(self, mb_id: int) -> torch.Tensor:
        """Value for ``mb_id`` once its transfer (if any) has completed, detached."""
        entry = self.get(self.to_process, mb_id)
        if entry == "remote":
            entry = self.recv_channel.wait(mb_id)
        return entry.detach()

    def clear(self) -> None:
        self.to_process.clear()
        self.saved.clear()
        self.to_send.clear()

    def __repr__(self) -> str:
        return f"Variable({self.name} <-> block {self.peer_id})"


class PipelineBlock:
    _step_counter = 0  # bumped by the pipeline at the start of every step (see all_reduce_param_grads)

    def __init__(self, model, id_, placement, signature, pp_group=None, dp_group=None, channels=None, device=None, rank=None):
        """``placement`` holds pipeline-local ranks; ``channels`` is this rank's
        ``ChannelTable`` (``None`` for a single-rank pipeline)."""
        self.id = id_
        self.placement = placement
        self.rank = placement[id_] if rank is None else rank
        if device is None:
            device = torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else torch.device("cpu")
        self.device = torch.device(device)
        self.model = model.to(self.device) if not any(p.is_meta for p in model.parameters()) else model
        self.is_first = id_ == 0
        self.is_last = id_ == len(placement) - 1
        self.pp_group = pp_group
        self.dp_group = dp_group
        self.signature = signature
        self.channels = channels
        self.input_variables: List[Variable] = [Variable(n, src, pp_group) for n, src in zip(signature.inputs, signature.sources)]
        self.output_variables: List[List[Variable]] = [
            [Variable(n, dst, pp_group) for dst in dsts] for n, dsts in zip(signature.outputs, signature.targets)
        ]
        self.compute_time: List = []
        self.remat_manager = RematManager(self)
        self._dw_layers: Optional[List[LayerDW]] = None
        self._grad_sync = None  # set by the pipeline: callable(block, batch_size)
        self._pending_reduce: List = []

    def __str__(self) -> str:
        return f"Rank {self.rank} - Layer {self.id}"

    __repr__ = __str__

    # ------------------------------------------------------------------ helpers
    def dw_layers(self) -> List[LayerDW]:
        if self._dw_layers is None:
            self._dw_layers = [m for m in self.model.modules() if isinstance(m, LayerDW)]
        return self._dw_layers

    def invalidate_layer_cache(self) -> None:
        self._dw_layers = None

    def _is_local(self, block_id: Optional[int]) -> bool:
        return block_id is not None and self.placement[block_id] == self.rank

    def _timed(self, name: str):
        timer = Timer(name=name)
        self.compute_time.append(timer)
        return timer

    def _run_forward(self, inputs, name: str):
        with self._timed(name):
            y = self.model(*inputs)
        return y if isinstance(y, tuple) else (y,)

    def _file_stashes(self, queue: str, mb_id: int) -> None:
        for layer in self.dw_layers():
            layer.move_last_computed(queue, mb_id)

    # ------------------------------------------------------------------ compute ops
    def forward(self, mb_id: int, **options):
        inputs = []
        for var in self.input_variables:
            x = var.wait_and_pop(mb_id)
            if x.is_floating_point() or x.is_complex():
                x.requires_grad_(True)
            inputs.append(x)

        strategy = options.get(OpOptions.REMAT_STRATEGY) or (lambda *_: False)
        with self.remat_manager.apply_selective_remat(strategy, mb_id):
            y = self._run_forward(inputs, f"forward({self.id}:{mb_id})")
            self._file_stashes("input", mb_id)

        for var_dsts, value in zip(self.output_variables, y):
            for var in var_dsts:
                if var.metadata is None:
                    var.metadata = TensorMetadata(shape=list(value.shape[1:]) if value.dim() else [], dtype=value.dtype, device=self.device)
                var.set(var.to_send, mb_id, value.detach())
            var_dsts[0].set(var_dsts[0].saved, mb_id, value)
        for var, value in zip(self.input_variables, inputs):
            var.set(var.saved, mb_id, value)

        if self.is_last:
            outs = []
            for var_dsts in self.output_variables:
                assert len(var_dsts) == 1, "Output of the pipeline has multiple destinations"
                outs.append(var_dsts[0].get(var_dsts[0].to_send, mb_id))
            return outs
        return None

    def backward_inputs(self, mb_id: int, **options):
        inputs = [v.get(v.saved, mb_id) for v in self.input_variables]
        outputs = [v[0].get(v[0].saved, mb_id) for v in self.output_variables]
        out_grads = []
        for var_dsts in self.output_variables:
            for var in var_dsts:  # gradient channels learn their shape from the forward output
                ch = var.recv_channel
                if ch is not None and ch.direction == "bwd" and ch.metadata is None and var.metadata is not None:
                    ch.set_metadata(var.metadata)
            g = var_dsts[0].wait_and_pop(mb_id)
            for other in var_dsts[1:]:
                g = g + other.wait_and_pop(mb_id)
            out_grads.append(g)

        drop_inputs = bool(options.get(OpOptions.RECOMPUTE_ACTIVATIONS, False))
        drop_grads = bool(options.get(OpOptions.RECOMPUTE_GRADIENTS, False))

        assert len(outputs) == len(out_grads)
        with self._timed(f"backward_inputs({self.id}:{mb_id})"):
            live = [(o, g) for o, g in zip(outputs, out_grads) if o.requires_grad]
            for o, g in live:
                assert o.shape == g.shape, f"Output and grad shapes do not match: {o.shape} != {g.shape}"
            if live:
                # one traversal for all outputs: shared nodes run their backward once (custom
                # functions that free their state on the first call rely on this)
                torch.autograd.backward([o for o, _ in live], [g.to(o.dtype) for o, g in live])

        in_grads = [x.grad.data if x.grad is not None else torch.zeros_like(x) for x in inputs if x.requires_grad]

        for layer in self.dw_layers():
            layer.move_last_computed("grad_output", mb_id)
            if drop_grads and len(layer.ctx["grad_output"]) > mb_id and layer.ctx["grad_output"][mb_id] is not None:
                layer.delete("grad_output", mb_id)
            if getattr(layer, "last_input", None) is not None:  # checkpoint re-ran the forward
                layer.move_last_computed("input", mb_id)
            if drop_inputs and len(layer.ctx["input"]) > mb_id and layer.ctx["input"][mb_id] is not None:
                layer.delete("input", mb_id)
        if options.get(OpOptions.OFFLOAD_DW, False):
            self._offload_dw(mb_id)

        grad_vars = [v for v, x in zip(self.input_variables, inputs) if x.requires_grad]
        for var, g in zip(grad_vars, in_grads):
            var.set(var.to_send, mb_id, g)
        if drop_inputs:  # the recompute-forward before W needs the stage inputs again
            for var, x in zip(self.input_variables, inputs):
                var.set(var.saved, mb_id, x.detach().requires_grad_(x.requires_grad))
        if drop_grads:
            for var_dsts, g in zip(self.output_variables, out_grads):
                var_dsts[0].set(var_dsts[0].to_process, mb_id, g)

    def backward_params(self, mb_id: int, **options):
        final = mb_id == getattr(self, "final_w_mb", None)
        with self._timed(f"backward_params({self.id}:{mb_id})"):
            for layer in self.dw_layers():
                slots = layer.ctx["grad_output"]
                if len(slots) > mb_id and slots[mb_id] is not None:
                    layer._final_pass = final  # last W of the step for this stage: gradients are complete
                    layer.backward(mb_id)

    def recompute_forward(self, mb_id: int, **options):
        inputs = [v.get(v.saved, mb_id) for v in self.input_variables]
        keep_graph = bool(options.get(OpOptions.SAVE, False))
        name = f"recompute_forward({self.id}:{mb_id})"
        if keep_graph:
            y = self._run_forward(inputs, name)
            for var, x in zip(self.input_variables, inputs):
                var.set(var.saved, mb_id, x)
            for var_dsts, value in zip(self.output_variables, y):
                var_dsts[0].set(var_dsts[0].saved, mb_id, value)
        else:
            with torch.no_grad():
                self._run_forward(inputs, name)
        self._file_stashes("input", mb_id)

    def recompute_backward_inputs(self, mb_id: int, **options):
        for v in self.input_variables:
            v.get(v.saved, mb_id)
        outputs = [v[0].get(v[0].saved, mb_id) for v in self.output_variables]
        grads = [v[0].get(v[0].to_process, mb_id) for v in self.output_variables]
        with self._timed(f"recompute_backward_inputs({self.id}:{mb_id})"):
            live = [(o, g) for o, g in zip(outputs, grads) if o.requires_grad]
            # only the part of the backward that reaches the split-backward layers
            if len(live) == 1:
                partial_dx_recomputation(live[0][0], live[0][1].to(live[0][0].dtype))
            elif live:
                partial_dx_recomputation([o for o, _ in live], [g.to(o.dtype) for o, g in live])
        self._file_stashes("grad_output", mb_id)

    def _offload_dw(self, mb_id: int, to="cpu") -> None:
        """Park the W-pass operands of ``mb_id`` on the host until ``backward_params``."""
        for layer in self.dw_layers():
            layer.offload_last(mb_id, to)

    # ------------------------------------------------------------------ communication ops
    def _out_var(self, dst) -> List[Variable]:
        return [v for var_dsts in self.output_variables for v in var_dsts if v.peer_id == dst]

    def _in_var(self, src) -> List[Variable]:
        return [v for v in self.input_variables if v.peer_id == src]

    def send_forward(self, mb_id: int, **options):
        dst = options.get("dst")
        if dst is None or self._is_local(dst):
            return  # pipeline output, or a same-rank hand-off done by the engine
        for k, var in enumerate(self._out_var(dst)):
            ch_k = self.channels.get(self.id, dst, "fwd", k)
            ch_k.send(var.get(var.to_send, mb_id), mb_id)

    def send_backward(self, mb_id: int, **options):
        dst = options.get("dst")
        if dst is None or self._is_local(dst):
            return
        for k, var in enumerate(self._in_var(dst)):
            ch_k = self.channels.get(self.id, dst, "bwd", k)
            if var.to_send.get(mb_id) is None:
                continue  # integer input: no gradient flows back
            ch_k.send(var.get(var.to_send, mb_id), mb_id)

    def recv_forward(self, mb_id: int, mb_size: int = 1, **options):
        src = options.get("src")
        if src is None or self._is_local(src):
            return
        for k, var in enumerate(self._in_var(src)):
            ch_k = self.channels.get(src, self.id, "fwd", k)
            var.recv_channel = ch_k
            ch_k.post_recv(mb_id, mb_size)
            var.set(var.to_process, mb_id, "remote")

    def recv_backward(self, mb_id: int, mb_size: int = 1, **options):
        src = options.get("src")
        if src is None or self._is_local(src):
            return
        for k, var in enumerate(self._out_var(src)):
            ch_k = self.channels.get(src, self.id, "bwd", k)
            if ch_k.metadata is None and var.metadata is not None:
                ch_k.set_metadata(var.metadata)  # a gradient has the shape of the tensor we sent
            var.recv_channel = ch_k
            ch_k.post_recv(mb_id, mb_size)
            var.set(var.to_process, mb_id, "remote")

    # ------------------------------------------------------------------ gradients
    def scale_grads(self, batch_size: int) -> None:
        """Divide every gradient by the number of samples of the step."""
        if batch_size == 1:
            return
        inv = 1.0 / batch_size
        for p in self.model.parameters():
            if p.grad is not None:
                p.grad.mul_(inv)

    def all_reduce_param_grads(self) -> None:
        """Average gradients over the data-parallel replicas holding this stage.  Work
        handles are kept and waited by ``wait_grad_sync`` (the reference drops them,
        ``elf/execution/block.py:514-516``)."""
        if self.dp_group is None or dist.get_world_size(self.dp_group) == 1:
            return
        world = dist.get_world_size(self.dp_group)
        avg_ok = dist.get_backend(self.dp_group) == "nccl"
        # parameters living in a flat buffer (the fused optimizer's): reduce the buffer in place, one
        # collective, no gather / scatter copies.  A buffer shared by several stages of this rank is
        # reduced once per step, by whichever stage gets here first (every W pass of the step is
        # done by then: the all-reduce operations close the schedule).
        loose = []
        for _, p in sorted(self.model.named_parameters(), key=lambda kv: kv[0]):
            group = getattr(p, "_elf_flat_group", None)
            if group is None or group.grad_dtype != p.dtype or p.grad is None or p.grad.data_ptr() != group.grad_view(group.params.index(p)).data_ptr():
                if p.grad is not None:
                    loose.append(p.grad)
                continue
            if getattr(group, "_reduced_in_step", None) == PipelineBlock._step_counter:
                continue
            group._reduced_in_step = PipelineBlock._step_counter
            work = dist.all_reduce(group.flat_grad, op=dist.ReduceOp.AVG if avg_ok else dist.ReduceOp.SUM, group=self.dp_group, async_op=True)
            self._pending_reduce.append((work, group.flat_grad, [], 1.0 if avg_ok else 1.0 / world))
        grads = loose
        if not grads:
            return
        by_dtype: Dict[torch.dtype, List[torch.Tensor]] = {}
        for g in grads:
            by_dtype.setdefault(g.dtype, []).append(g)
        for bucket in by_dtype.values():
            flat = torch.cat([g.reshape(-1) for g in bucket])
            work = dist.all_reduce(flat, op=dist.ReduceOp.AVG if avg_ok else dist.ReduceOp.SUM, group=self.dp_group, async_op=True)
            self._pending_reduce.append((work, flat, bucket, 1.0 if avg_ok else 1.0 / world))

    def sync_grads(self, batch_size: int) -> None:
        """ALL_REDUCE_PARAM_GRADS: 1/batch scaling followed by the DP average."""
        if self._grad_sync is not None:
            self._grad_sync(self, batch_size)
            return
        self.scale_grads(batch_size)
        self.all_reduce_param_grads()

    def wait_grad_sync(self) -> None:
        for work, flat, bucket, factor in self._pending_reduce:
            work.wait()
            if not bucket:  # a flat gradient buffer reduced in place
                if factor != 1.0:
                    flat.mul_(factor)
                continue
            offset = 0
            for g in bucket:
                n = g.numel()
                chunk = flat[offset : offset + n].view_as(g)
                g.copy_(chunk if factor == 1.0 else chunk * factor)
                offset += n
        self._pending_reduce.clear()

    # ------------------------------------------------------------------ housekeeping
    def clear_slots(self) -> None:
        for var in self.input_variables:
            var.clear()
        for var_dsts in self.output_variables:
            for var in var_dsts:
                var.clear()
        for layer in self.dw_layers():
            layer.clear()

    def _wait_for_send_ops(self) -> None:
        if self.channels is not None:
            for ch in self.channels.channels.values():
                ch.reap_sends()

    def _destroy_process_groups(self) -> None:
        if self.channels is not None:
            self.channels.destroy()
