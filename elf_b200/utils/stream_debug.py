"""Debug mode for stream ordering: which stream last wrote a buffer, and did its reader wait?

The runtime moves tensors between CUDA streams in a handful of places (activation offload
and prefetch, results copied to the host, the copy-engine transport between stages).  Each
hand-off needs a ``wait_stream`` / ``wait_event`` on the consumer's side; a missing one is a
race that usually passes unnoticed.  With ``ELF_B200_DEBUG_STREAMS=1`` those places report
what they do to this module, which keeps a logical clock and checks, on the host and
without touching the GPU:

``note_write(tensor, stream)``  the stream has been given work that writes the tensor's storage
``note_sync(consumer, producer)``  consumer-stream work issued from now on runs after everything
                                   issued so far on the producer stream (``wait_stream`` / a waited event)
``check_read(tensor, stream)``  work reading the storage is about to be issued on ``stream``:
                                raises ``StreamOrderError`` if another stream wrote it more
                                recently than the reader last synchronised with that stream

Streams are identified by any hashable key (``stream.cuda_stream`` for CUDA streams, plain
strings in tests), storages by ``untyped_storage().data_ptr()``.  The checker has no
counterpart in the reference, which relies on convention (``record_stream`` on offloaded
sources, event waits before prefetched data is used; ``elf/execution/offload.py:285-341``).
"""

from __future__ import annotations

import os
from typing import Dict, Hashable, Tuple

__all__ = ["StreamOrderError", "enabled", "enable", "reset", "note_write", "note_sync", "check_read", "stream_key"]


class StreamOrderError(RuntimeError):
    pass


_enabled = os.environ.get("ELF_B200_DEBUG_STREAMS", "0") not in ("", "0", "false", "no")
_clock = 0
_last_write: Dict[int, Tuple[Hashable, int, str]] = {}  # storage -> (stream, time, note)
_synced: Dict[Tuple[Hashable, Hashable], int] = {}  # (consumer, producer) -> time of the last sync


def enabled() -> bool:
    return _enabled


def enable(flag: bool = True) -> None:
    global _enabled
    _enabled = bool(flag)
    reset()


def reset() -> None:
    global _clock
    _clock = 0
    _last_write.clear()
    _synced.clear()


def stream_key(stream) -> Hashable:
    """Key of a ``torch.cuda.Stream`` (or of anything hashable passed as a stand-in)."""
    return getattr(stream, "cuda_stream", stream)


def _storage_key(tensor) -> int:
    try:
        return tensor.untyped_storage().data_ptr()
    except Exception:
        return id(tensor)


def _tick() -> int:
    global _clock
    _clock += 1
    return _clock


def note_write(tensor, stream, note: str = "") -> None:
    if not _enabled:
        return
    _last_write[_storage_key(tensor)] = (stream_key(stream), _tick(), note)


def note_sync(consumer, producer) -> None:
    if not _enabled:
        return
    _synced[(stream_key(consumer), stream_key(producer))] = _tick()


def check_read(tensor, stream, note: str = "") -> None:
    if not _enabled:
        return
    entry = _last_write.get(_storage_key(tensor))
    if entry is None:
        return
    writer, when, what = entry
    reader = stream_key(stream)
    if writer == reader:
        return
    if _synced.get((reader, writer), 0) < when:
        raise StreamOrderError(
            f"stream {reader!r} reads a buffer ({note or 'unnamed'}) that stream {writer!r} wrote ({what or 'unnamed'}) "
            "without having waited for that stream since: a wait_stream / wait_event is missing"
        )
