"""Data-parallel gradient synchronisation over NVLink peer memory, fused with the
weight-gradient GEMM.

The reference averages gradients with one NCCL ``all_reduce`` per parameter tensor after the
last W pass of the step, with nothing overlapped (``elf/execution/block.py:506-527``).  Here:

* each stage's bf16 parameters and gradients live in flat buffers (``FlatGroup``);
* every replica owns an *inbox* in symmetric memory: two parities x (R-1) slots of the
  gradient buffer's size, plus 32-bit flags;
* the LAST weight-gradient GEMM of a step for a matrix runs with a push target: its epilogue
  stores the finished tile locally **and** into this replica's slot of every peer's inbox
  (plain stores to peer memory from the tcgen05 kernel), and the last CTA of the launch
  raises that matrix's flag on the peers - so the exchange of a layer's gradient overlaps
  the remaining B / F / W passes of the schedule;
* at the step's ALL_REDUCE op everything the GEMMs did not push (norm gains, embedding,
  matrices whose gradient did not come from the split backward) is pushed by one copy
  kernel, and one finalize kernel waits (bounded) for the peers' flags and leaves
  ``scale * (local + sum of peers)`` in the local gradient buffer.

No NCCL call and no library GEMM is on that path.  Each replica sends (R-1) copies of its
gradient, which is bandwidth-optimal for R = 2 (the configuration the benchmarks name) and
1.5x the reduce-scatter + all-gather volume for R = 4.
"""

from __future__ import annotations

import logging
from typing import Dict, List, Optional, Sequence

import torch
import torch.distributed as dist

from ..ops import _ext
from ..ops import gemm as _gemm
from ..optim.flat import FlatGroup
from ..zb_utils import LinearDW
from .symm import SymmetricBuffer

logger = logging.getLogger("dp_sync")

__all__ = ["SymmetricGradSync", "StageExchange", "LayerPush"]


class LayerPush:
    """Push description of one matrix: where it sits in the flat gradient buffer and which
    flag announces it."""

    def __init__(self, exchange: "StageExchange", offset: int, flag_index: int):
        self.exchange, self.offset, self.flag_index = exchange, offset, flag_index

    def target(self) -> Optional[dict]:
        ex = self.exchange
        if not ex.armed:
            return None
        ex.pushed.add(self.flag_index)
        byte_off = ex.parity_offset_bytes() + self.offset * 2
        return {
            "push_out": [base + byte_off for base in ex.peer_slot_addr],
            "push_flags": [base + 4 * self.flag_index for base in ex.peer_flag_addr],
            "push_flag_value": ex.epoch,
            "push_counter": ex.counter,
        }


class StageExchange:
    """Flat gradient buffer, inbox and flags of ONE stage on ONE replica."""

    def __init__(self, flat: FlatGroup, inbox: SymmetricBuffer, flags: SymmetricBuffer, rank: int, world: int, timeout_ms: float = 30000.0):
        self.flat, self.inbox, self.flags = flat, inbox, flags
        self.rank, self.world = rank, world
        self.n_peers = world - 1
        self.numel = flat.numel
        self.timeout_ms = timeout_ms
        dev = flat.device
        self.matrices: List[LayerPush] = []
        self.n_flags = 1  # flag 0 announces the "rest" copy
        self.epoch = 0
        self.armed = False
        self.pushed = set()
        self.counter = torch.zeros(1, dtype=torch.int32, device=dev)
        self.status = _gemm.status(dev)
        self._tables: Dict[int, tuple] = {}
        self._peers = [p for p in range(world) if p != rank]
        # my slot on peer p is indexed by my rank among p's peers
        self._slot_on = {p: (rank if rank < p else rank - 1) for p in self._peers}

    def finish_layout(self) -> None:
        """Call once all matrices are registered: sizes the flag array addressing."""
        slot_bytes = self.numel * 2
        self.parity_stride_bytes = self.n_peers * slot_bytes
        self.peer_slot_addr = [self.inbox.peer_address(p, self._slot_on[p] * slot_bytes) for p in self._peers]
        self.peer_flag_addr = [self.flags.peer_address(p, self._slot_on[p] * self.n_flags * 4) for p in self._peers]

    def register_matrix(self, offset: int) -> LayerPush:
        lp = LayerPush(self, offset, self.n_flags)
        self.n_flags += 1
        self.matrices.append(lp)
        return lp

    def parity_offset_bytes(self) -> int:
        return (self.epoch & 1) * self.parity_stride_bytes

    # ------------------------------------------------------------------ per step
    def begin_step(self) -> None:
        self.epoch += 1
        self.pushed = set()
        self.armed = True

    def _device_tables(self):
        key = self.epoch & 1
        if key not in self._tables:
            dev = self.flat.device
            off = key * self.parity_stride_bytes
            slots = torch.tensor([a + off for a in self.peer_slot_addr], dtype=torch.int64, device=dev)
            flags = torch.tensor(self.peer_flag_addr, dtype=torch.int64, device=dev)  # flag 0 of my slot on each peer
            self._tables[key] = (slots, flags)
        return self._tables[key]

    def finish_step(self, scale: float) -> None:
        """Push what the GEMM epilogues did not, then reduce.  Enqueues two kernels."""
        self.push_rest()
        self.reduce(scale)

    def push_rest(self) -> None:
        """Copy every range no GEMM epilogue pushed into the peers' inboxes and raise flag 0."""
        ext = _ext.get()
        dev = self.flat.device
        self.flat.gather_stray_grads()
        covered = sorted((m.offset, m.offset + self._matrix_numel(m)) for m in self.matrices if m.flag_index in self.pushed)
        ranges, cursor = [], 0
        for b, e in covered:
            if b > cursor:
                ranges.append((cursor, b))
            cursor = max(cursor, e)
        if cursor < self.numel:
            ranges.append((cursor, self.numel))
        slots, flags = self._device_tables()
        rng = torch.tensor(ranges if ranges else [(0, 0)], dtype=torch.int64, device=dev)
        ext.push_ranges(self.flat.flat_grad, rng, slots, flags, self.epoch, self.counter)

    def reduce(self, scale: float) -> None:
        """Wait (bounded) for the peers' flags of this step, then ``grad = scale * (local + peers)``."""
        ext = _ext.get()
        dev = self.flat.device
        wait = torch.tensor([0] + sorted(self.pushed), dtype=torch.int32, device=dev)
        par = self.epoch & 1
        inbox = self.inbox.local[par * self.n_peers * self.numel : (par + 1) * self.n_peers * self.numel]
        ext.finalize_reduce(self.flat.flat_grad, inbox, self.n_peers, self.flags.local, self.n_flags, wait, self.epoch, scale, self.timeout_ms, self.status)
        self.armed = False

    def _matrix_numel(self, m: LayerPush) -> int:
        return self._sizes[m.flag_index]

    _sizes: Dict[int, int]


def _build_exchange(params: Sequence[torch.nn.Parameter], layers: Sequence[LinearDW], allocate, rank: int, world: int, timeout_ms: float) -> Optional[StageExchange]:
    params = [p for p in params if p.requires_grad and p.is_cuda and p.dtype == torch.bfloat16]
    if not params:
        return None
    flat = FlatGroup(params)
    offsets = {id(p): off for p, off in zip(flat.params, flat.offsets)}
    n_matrices = sum(1 for l in layers if id(l.weight) in offsets)
    inbox = allocate(2 * (world - 1) * flat.numel, torch.bfloat16)
    flags = allocate((world - 1) * (1 + n_matrices), torch.int32)
    ex = StageExchange(flat, inbox, flags, rank, world, timeout_ms)
    ex._sizes = {}
    for layer in layers:
        off = offsets.get(id(layer.weight))
        if off is None:
            continue
        lp = ex.register_matrix(off)
        ex._sizes[lp.flag_index] = layer.weight.numel()
        layer._push = lp
    ex.finish_layout()
    return ex


class SymmetricGradSync:
    """Callable installed as ``block._grad_sync``; owns one ``StageExchange`` per local stage."""

    def __init__(self, blocks, dp_group, timeout_ms: float = 30000.0):
        _ext.require_on_gpu()
        if not hasattr(_ext.get(), "push_ranges"):
            raise RuntimeError("extension built without the dp_reduce kernels")
        self.group = dp_group
        self.rank = dist.get_rank(dp_group)
        self.world = dist.get_world_size(dp_group)
        if self.world - 1 > 7:
            raise RuntimeError("peer push supports at most 8 replicas")
        self.exchanges: Dict[int, Optional[StageExchange]] = {}
        for block in blocks:
            alloc = lambda n, dt: SymmetricBuffer.allocate(n, dt, dp_group, block.device)
            layers = [m for m in block.model.modules() if isinstance(m, LinearDW)]
            self.exchanges[block.id] = _build_exchange(list(block.model.parameters()), layers, alloc, self.rank, self.world, timeout_ms)

    def begin_step(self) -> None:
        for ex in self.exchanges.values():
            if ex is not None:
                ex.begin_step()

    def __call__(self, block, batch_size: int) -> None:
        ex = self.exchanges.get(block.id)
        scale = 1.0 / (batch_size * self.world)
        if ex is not None:
            ex.finish_step(scale)
        in_flat = {id(p) for p in ex.flat.params} if ex is not None else set()
        rest = [p for p in block.model.parameters() if p.grad is not None and id(p) not in in_flat]
        for p in rest:  # fp32 / CPU leftovers: plain collective
            p.grad.mul_(1.0 / batch_size)
            dist.all_reduce(p.grad, op=dist.ReduceOp.AVG, group=self.group)

    def close(self) -> None:
        self.exchanges.clear()
