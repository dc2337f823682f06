"""Context-manager timers returning seconds (reference ``elf/utils.py:249-324``)."""

from __future__ import annotations

import time

import torch

__all__ = ["Timer", "TimerCPU", "TimerGPU"]


class TimerCPU:
    def __init__(self, name: str = "unknown"):
        self.name = name
        self.start = self.end = 0.0

    def __enter__(self):
        self.start = time.perf_counter()
        return self

    def __exit__(self, *_):
        self.end = time.perf_counter()

    def time(self) -> float:
        return self.end - self.start


class TimerGPU:
    """CUDA-event timer on the current stream. ``time()`` blocks on the end event."""

    def __init__(self, name: str = "unknown"):
        self.name = name
        self.start_event = torch.cuda.Event(enable_timing=True)
        self.end_event = torch.cuda.Event(enable_timing=True)

    def __enter__(self):
        self.start_event.record()
        return self

    def __exit__(self, *_):
        self.end_event.record()

    def time(self) -> float:
        self.end_event.synchronize()
        return self.start_event.elapsed_time(self.end_event) / 1e3


class Timer:
    """Factory: ``Timer("gpu"|"cuda"|"cpu", name)``; with no type, GPU when CUDA exists."""

    def __new__(cls, type=None, name=None, *, type_=None, name_=None):
        kind = (type or type_ or "").lower()
        label = name or name_ or "unknown"
        if kind in ("gpu", "cuda"):
            return TimerGPU(label)
        if kind == "cpu":
            return TimerCPU(label)
        return TimerGPU(label) if torch.cuda.is_available() else TimerCPU(label)
