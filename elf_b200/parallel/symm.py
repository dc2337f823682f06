"""Symmetric memory: buffers that every rank of a group allocates at the same size and that
every other rank of the group can address directly over NVLink.

Two providers, chosen with ``ELF_B200_SYMM``:

``torch`` (default)  allocation, handle exchange and peer mapping by
                     ``torch.distributed._symmetric_memory`` (CUDA virtual-memory handles exchanged
                     through the group's store);
``vmm``              this package's own runtime (``csrc/symm_runtime.cpp``): every rank creates one
                     physical allocation with the CUDA virtual-memory API, exports it as a file
                     descriptor, the descriptors travel between the processes of the node over
                     UNIX-domain sockets (``SCM_RIGHTS``), and every rank maps its peers'
                     allocations.  No multicast object is bound: the consumers here (gradient push,
                     stage-to-stage rings) are point-to-point stores.

What this module adds on top is the view the kernels need: raw peer addresses, and a
single-process stand-in (``LocalSymmetricGroup``) in which several *virtual ranks* live on one
GPU so that the push/finalize protocol can be exercised end to end on one device (kernels that
never wait on a later launch are safe to run back to back).
"""

from __future__ import annotations

import os
import socket
import tempfile
import threading
import uuid
from typing import List, Sequence

import torch
import torch.distributed as dist

__all__ = ["SymmetricBuffer", "LocalSymmetricGroup", "exchange_fds"]


class SymmetricBuffer:
    """``local`` tensor + the device address of the same buffer on every rank of the group."""

    def __init__(self, local: torch.Tensor, addresses: Sequence[int], rank: int):
        self.local = local
        self.addresses = [int(a) for a in addresses]
        self.rank = rank
        self.world = len(self.addresses)

    @staticmethod
    def allocate(numel: int, dtype: torch.dtype, group, device=None) -> "SymmetricBuffer":
        device = device if device is not None else torch.device("cuda", torch.cuda.current_device())
        if os.environ.get("ELF_B200_SYMM", "torch") == "vmm":
            return _allocate_vmm(numel, dtype, group, device)
        import torch.distributed._symmetric_memory as symm_mem

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

    def peer_bytes(self, peer: int) -> torch.Tensor:
        """The buffer of rank ``peer`` as a uint8 tensor on this device (a mapping of the peer's
        memory: copies into it cross NVLink)."""
        nbytes = self.local.numel() * self.local.element_size()
        if peer == self.rank:
            return self.local.view(torch.uint8)
        handle = getattr(self, "_handle", None)
        if handle is None:
            raise RuntimeError("this buffer has no peer mappings (single-process stand-in)")
        if hasattr(handle, "peer_tensor"):  # own runtime: mappings are numbered in import order, i.e. by rank without this one
            return handle.peer_tensor(peer if peer < self.rank else peer - 1)[:nbytes]
        return handle.get_buffer(peer, (nbytes,), torch.uint8)


def exchange_fds(my_fd: int, group) -> List[int]:
    """Give every other rank of ``group`` (processes of one node) a duplicate of ``my_fd`` and return
    theirs, indexed by group rank (``-1`` at this rank's own index).  Each rank listens on a
    UNIX-domain socket whose path the ranks publish with ``all_gather_object``; descriptors cross
    as ancillary data (``SCM_RIGHTS``), which is how a CUDA allocation exported as a POSIX file
    descriptor reaches the process that imports it."""
    rank, world = dist.get_rank(group), dist.get_world_size(group)
    path = os.path.join(tempfile.gettempdir(), f"elf_b200_symm_{uuid.uuid4().hex}_{rank}.sock")
    server = socket.socket(socket.AF_UNIX, socket.SOCK_STREAM)
    server.bind(path)
    server.listen(world)
    received: List[int] = [-1] * world
    errors: List[BaseException] = []

    def accept_all():
        try:
            for _ in range(world - 1):
                conn, _addr = server.accept()
                with conn:
                    msg, fds, _flags, _a = socket.recv_fds(conn, 16, 1)
                    received[int(msg.decode())] = fds[0]
        except BaseException as exc:  # surfaced on the caller's thread below
            errors.append(exc)

    listener = threading.Thread(target=accept_all, daemon=True)
    listener.start()
    try:
        paths: List[str] = [""] * world
        dist.all_gather_object(paths, path, group=group)
        for peer in range(world):
            if peer == rank:
                continue
            with socket.socket(socket.AF_UNIX, socket.SOCK_STREAM) as conn:
                conn.connect(paths[peer])
                socket.send_fds(conn, [str(rank).encode()], [my_fd])
        listener.join(timeout=120)
        if listener.is_alive() or errors:
            raise RuntimeError(f"exchange of memory handles did not complete: {errors[0] if errors else 'a peer never connected'}")
    finally:
        server.close()
        try:
            os.unlink(path)
        except OSError:
            pass
    return received


def _allocate_vmm(numel: int, dtype: torch.dtype, group, device) -> "SymmetricBuffer":
    """``SymmetricBuffer.allocate`` on this package's own runtime (``VmmArena``)."""
    from ..ops import _ext

    ext = _ext.get()
    rank, world = dist.get_rank(group), dist.get_world_size(group)
    nbytes = numel * torch.empty(0, dtype=dtype).element_size()
    arena = ext.VmmArena(nbytes, device.index if device.index is not None else torch.cuda.current_device())
    fd = arena.export_fd()
    try:
        theirs = exchange_fds(fd, group)
    finally:
        os.close(fd)
    addresses = [0] * world
    try:
        for peer in range(world):
            if peer == rank:
                addresses[peer] = arena.address
                continue
            fd, theirs[peer] = theirs[peer], -1  # import_peer closes the descriptor, whatever happens
            addresses[peer] = arena.peer_address(arena.import_peer(fd))
    finally:
        for fd in theirs:  # descriptors that were never imported (an earlier import failed)
            if fd >= 0:
                os.close(fd)
    local = arena.tensor()[:nbytes].view(dtype)
    buf = SymmetricBuffer(local, addresses, rank)
    buf._handle = arena  # owns the allocation and the peer mappings
    torch.cuda.synchronize(device)
    dist.barrier(group=group)  # nobody touches a peer's buffer before every rank has mapped it
    return buf


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
