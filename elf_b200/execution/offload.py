"""Activation offload to pinned host memory.

``OffloadToCPU`` is a ``saved_tensors_hooks`` context: tensors autograd saves during a
forward are copied to pinned host memory on a device→host stream and replaced by a light
record; ``prefetch()`` starts the host→device copies on a second stream ahead of the
backward; the unpack hook waits for the copy (or performs it synchronously) and rebuilds
the original view.  Rules kept from the reference (``elf/execution/offload.py:166-411``):
tensors of at most 1 MiB, CPU tensors and excluded storages (parameters) are passed
through untouched; tensors that view one storage share one host copy of the used span.

Differences: the two side streams and the pinned arena belong to one ``OffloadManager``
per engine and are shared by all (stage, micro-batch) offloaders, instead of two new CUDA
streams per offloader per step (``elf/execution/engine.py:172-177``); host memory comes
from the native ``PinnedArena`` (first fit, coalescing); everything degrades to plain
synchronous copies on a CPU-only machine so the logic is testable without a GPU.
"""

from __future__ import annotations

import logging
from typing import Any, Dict, Iterable, Optional
from weakref import ref

import torch

from ..utils import stream_debug as _sd

from ..ops import _ext

logger = logging.getLogger("offload")

__all__ = ["PinnedHostTensorPool", "OffloadToCPU", "OffloadManager", "MIN_OFFLOAD_BYTES"]

MIN_OFFLOAD_BYTES = 1 << 20


class PinnedHostTensorPool:
    """Pool of pinned host tensors: ``allocate(numel, dtype)`` → 1-D tensor, ``free(t)``,
    ``reserve(bytes, dtype)``, ``size()`` (reference ``elf/execution/offload.py:14-163``).

    Backed by the native arena (``elf_b200/csrc/host_runtime.cpp``); dtype does not
    partition the arena.  Without the extension, falls back to ``torch.empty(pin_memory=)``."""

    def __init__(self, min_block_bytes: int = 64 << 20):
        self._arena = _ext.get().PinnedArena(min_block_bytes) if _ext.available() else None
        self._live: Dict[int, int] = {}  # data_ptr -> arena address
        self._fallback_bytes = 0

    def reserve(self, nbytes: int, dtype: torch.dtype = torch.uint8) -> None:
        if self._arena is not None and nbytes > 0:
            self._arena.reserve(int(nbytes))

    def allocate(self, numel: int, dtype: torch.dtype) -> torch.Tensor:
        nbytes = max(1, numel) * torch.empty(0, dtype=dtype).element_size()
        if self._arena is None:
            self._fallback_bytes += nbytes
            return torch.empty(numel, dtype=dtype, pin_memory=torch.cuda.is_available())
        addr = self._arena.allocate(nbytes)
        t = _ext.get().host_tensor(addr, nbytes).view(dtype)[:numel]
        self._live[t.data_ptr()] = addr
        return t

    def free(self, t: torch.Tensor) -> None:
        addr = self._live.pop(t.data_ptr(), None)
        if addr is not None:
            self._arena.release(addr)

    def size(self) -> int:
        """Bytes of host memory held by the pool."""
        return self._arena.capacity if self._arena is not None else self._fallback_bytes

    @property
    def in_use(self) -> int:
        return self._arena.in_use if self._arena is not None else 0

    @property
    def peak(self) -> int:
        return self._arena.peak if self._arena is not None else 0


class OffloadManager:
    """Streams + arena shared by the offloaders of one engine."""

    def __init__(self, device=None, pool: Optional[PinnedHostTensorPool] = None):
        self.device = torch.device(device) if device is not None else torch.device("cpu")
        self.on_cuda = self.device.type == "cuda"
        self.pool = pool or PinnedHostTensorPool()
        self.d2h_stream = torch.cuda.Stream(self.device) if self.on_cuda else None
        self.h2d_stream = torch.cuda.Stream(self.device) if self.on_cuda else None
        self.bytes_offloaded = 0

    def offloader(self, exclude: Iterable[torch.Tensor] = ()) -> "OffloadToCPU":
        off = OffloadToCPU(pool=self.pool, manager=self)
        off.exclude(exclude)
        return off

    def finish_step(self, offloaders: Iterable["OffloadToCPU"]) -> None:
        """End of step: the compute stream waits for outstanding copies; host blocks go
        back to the arena."""
        offloaders = list(offloaders)
        if self.on_cuda and offloaders:
            cur = torch.cuda.current_stream(self.device)
            cur.wait_stream(self.d2h_stream)
            cur.wait_stream(self.h2d_stream)
        for off in offloaders:
            off.release()


class OffloadToCPU:
    """>>> with OffloadToCPU() as off:
    ...     loss = loss_fn(model(x))
    >>> off.prefetch()          # optional, some ops before the backward
    >>> loss.backward()
    >>> off.release()
    """

    def __init__(self, target_device="cpu", pool: Optional[PinnedHostTensorPool] = None, manager: Optional[OffloadManager] = None, min_bytes: int = MIN_OFFLOAD_BYTES):
        self.target_device = torch.device(target_device)
        if manager is None:
            dev = torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else torch.device("cpu")
            manager = OffloadManager(dev, pool)
        self._mgr = manager
        self._pool = pool or manager.pool
        self.min_bytes = min_bytes
        self._host: Dict[Any, torch.Tensor] = {}  # storage weakref -> flat host copy
        self._span: Dict[Any, int] = {}
        self._origin: Dict[Any, torch.device] = {}
        self._on_device: Dict[Any, torch.Tensor] = {}
        self._d2h_done: Dict[Any, Any] = {}
        self._h2d_done: Dict[Any, Any] = {}
        self._excluded = set()
        self._hooks = None
        self._copied_bytes = 0

    # A storage is identified by a weak reference to the storage *object*: a data pointer
    # could be recycled for another tensor once the original is freed — which is the
    # whole point of offloading.
    @staticmethod
    def _key(t: torch.Tensor):
        return ref(t.untyped_storage())

    def exclude(self, tensors: Iterable[torch.Tensor]) -> None:
        self._excluded.update(self._key(t) for t in tensors)

    # ------------------------------------------------------------------ hooks
    def _pack(self, t: torch.Tensor):
        if t.device.type == "cpu" and self._mgr.on_cuda:
            return t
        if t.nbytes <= self.min_bytes or t.is_meta:
            return t
        key = self._key(t)
        if key in self._excluded:
            return t
        offset = int(t.storage_offset())
        span = offset + 1 + sum((int(n) - 1) * int(st) for n, st in zip(t.size(), t.stride()) if n > 0)
        if any(st < 0 for st in t.stride()):
            return t
        if key not in self._host or span > self._span[key]:
            old = self._host.get(key)
            if old is not None:
                self._pool.free(old)
            host = self._pool.allocate(span, t.dtype)
            self._copy_out(host, t, span, key)
            self._host[key] = host
            self._span[key] = span
            self._origin[key] = t.device
        return {"key": key, "size": tuple(t.size()), "stride": tuple(t.stride()), "offset": offset, "dtype": t.dtype, "device": t.device}

    def _copy_out(self, host: torch.Tensor, src: torch.Tensor, span: int, key) -> None:
        flat = torch.as_strided(src.detach(), (span,), (1,), 0)
        mgr = self._mgr
        if mgr.on_cuda and src.is_cuda:
            cur = torch.cuda.current_stream(src.device)
            _sd.note_write(src, cur, "activation saved for backward")
            mgr.d2h_stream.wait_stream(cur)
            _sd.note_sync(mgr.d2h_stream, cur)
            _sd.check_read(src, mgr.d2h_stream, "offload copy to the host")
            with torch.cuda.stream(mgr.d2h_stream):
                host.copy_(flat, non_blocking=True)
                src.record_stream(mgr.d2h_stream)  # keep the device memory alive until copied
                ev = torch.cuda.Event()
                ev.record(mgr.d2h_stream)
            self._d2h_done[key] = ev
        else:
            host.copy_(flat)
        self._copied_bytes += flat.nbytes
        mgr.bytes_offloaded += flat.nbytes

    def _unpack(self, rec):
        if isinstance(rec, torch.Tensor):
            return rec
        key = rec["key"]
        base = self._on_device.get(key)
        if base is None:
            host = self._host[key]
            ev = self._d2h_done.get(key)
            if ev is not None:
                torch.cuda.current_stream(rec["device"]).wait_event(ev)
            base = host.to(rec["device"], non_blocking=False)
            self._on_device[key] = base
        ev = self._h2d_done.get(key)
        if ev is not None:
            torch.cuda.current_stream(rec["device"]).wait_event(ev)
            _sd.note_sync(torch.cuda.current_stream(rec["device"]), self._mgr.h2d_stream)
        if base.is_cuda:
            _sd.check_read(base, torch.cuda.current_stream(rec["device"]), "prefetched activation used by the backward")
        return torch.as_strided(base, rec["size"], rec["stride"], rec["offset"])

    # ------------------------------------------------------------------ prefetch / release
    def prefetch(self) -> None:
        """Start copying every offloaded storage back to its device."""
        mgr = self._mgr
        for key, host in list(self._host.items()):
            if key in self._on_device:
                continue
            dev = self._origin.get(key, mgr.device)
            if not (mgr.on_cuda and dev.type == "cuda"):
                self._on_device[key] = host.to(dev)
                continue
            # allocate on the compute stream (so the caching allocator orders reuse there),
            # copy on the h2d stream once the d2h copy of the same storage has finished
            buf = torch.empty(host.shape, dtype=host.dtype, device=dev)
            mgr.h2d_stream.wait_stream(torch.cuda.current_stream(dev))
            ev = self._d2h_done.get(key)
            if ev is not None:
                mgr.h2d_stream.wait_event(ev)
            with torch.cuda.stream(mgr.h2d_stream):
                buf.copy_(host, non_blocking=True)
                _sd.note_write(buf, mgr.h2d_stream, "prefetch copy from the host")
                done = torch.cuda.Event()
                done.record(mgr.h2d_stream)
            self._on_device[key] = buf
            self._h2d_done[key] = done

    def release(self) -> None:
        """Forget everything and give host blocks back to the pool."""
        if self._mgr.on_cuda and self._h2d_done:
            torch.cuda.current_stream(self._mgr.device).wait_stream(self._mgr.h2d_stream)
        if self._mgr.on_cuda and self._d2h_done:
            # a host block may be reused by the next allocation: its copy must have landed
            self._mgr.d2h_stream.synchronize()
        for host in self._host.values():
            self._pool.free(host)
        for table in (self._host, self._span, self._origin, self._on_device, self._d2h_done, self._h2d_done):
            table.clear()
        self._copied_bytes = 0

    @property
    def offloaded_bytes(self) -> int:
        return self._copied_bytes

    # ------------------------------------------------------------------ context manager
    def __enter__(self) -> "OffloadToCPU":
        self._hooks = torch.autograd.graph.saved_tensors_hooks(self._pack, self._unpack)
        self._hooks.__enter__()
        return self

    def __exit__(self, exc_type, exc, tb):
        if self._hooks is not None:
            self._hooks.__exit__(exc_type, exc, tb)
            self._hooks = None
        return False
