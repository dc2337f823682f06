"""Symmetric memory: buffers that every rank of a group allocates at the same size and that
every other rank of the group can address directly over NVLink.

Allocation, handle exchange and peer mapping are delegated to
``torch.distributed._symmetric_memory`` (CUDA virtual-memory handles exchanged through the
group's store).  What this module adds is the view the kernels need: raw peer addresses,
and a single-process stand-in (``LocalSymmetricGroup``) in which several *virtual ranks*
live on one GPU so that the push/finalize protocol can be exercised end to end on one
device (kernels that never wait on a later launch are safe to run back to back).
"""

from __future__ import annotations

from typing import List, Sequence

import torch
import torch.distributed as dist

__all__ = ["SymmetricBuffer", "LocalSymmetricGroup"]


class SymmetricBuffer:
    """``local`` tensor + the device address of the same buffer on every rank of the group."""

    def __init__(self, local: torch.Tensor, addresses: Sequence[int], rank: int):
        self.local = local
        self.addresses = [int(a) for a in addresses]
        self.rank = rank
        self.world = len(self.addresses)

    @staticmethod
    def allocate(numel: int, dtype: torch.dtype, group, device=None) -> "SymmetricBuffer":
        import torch.distributed._symmetric_memory as symm_mem

        device = device if device is not None else torch.device("cuda", torch.cuda.current_device())
        t = symm_mem.empty(numel, dtype=dtype, device=device)
        handle = symm_mem.rendezvous(t, group=group.group_name if hasattr(group, "group_name") else group)
        t.zero_()
        buf = SymmetricBuffer(t, list(handle.buffer_ptrs), handle.rank)
        buf._handle = handle  # keeps the mapping alive
        torch.cuda.synchronize(device)
        dist.barrier(group=group)
        return buf

    def peer_address(self, peer: int, byte_offset: int = 0) -> int:
        return self.addresses[peer] + byte_offset


class LocalSymmetricGroup:
    """``world`` virtual ranks on one device; ``allocate`` returns one buffer per rank, each
    knowing the addresses of all of them."""

    def __init__(self, world: int, device=None):
        self.world = world
        self.device = device if device is not None else torch.device("cuda", torch.cuda.current_device())

        self._sets: List[List[SymmetricBuffer]] = []
        self._next = [0] * world

    def allocate(self, numel: int, dtype: torch.dtype) -> List[SymmetricBuffer]:
        tensors = [torch.zeros(numel, dtype=dtype, device=self.device) for _ in range(self.world)]
        addrs = [t.data_ptr() for t in tensors]
        return [SymmetricBuffer(t, addrs, r) for r, t in enumerate(tensors)]

    def allocator(self, rank: int):
        """``allocate(numel, dtype)`` for virtual rank ``rank``: the k-th call of every rank
        returns that rank's member of the k-th symmetric set (as a collective would)."""

        def allocate(numel: int, dtype: torch.dtype) -> SymmetricBuffer:
            k = self._next[rank]
            self._next[rank] += 1
            if k == len(self._sets):
                self._sets.append(self.allocate(numel, dtype))
            buf = self._sets[k][rank]
            assert buf.local.numel() == numel and buf.local.dtype == dtype, "virtual ranks must allocate identically"
            return buf

        return allocate
