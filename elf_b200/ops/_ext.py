"""Locate and load the compiled extension (``elf_b200/csrc/_build/elf_b200_C.so``, or its
bounds-checking variant ``elf_b200/csrc/_build_check/elf_b200_C_check.so``)."""

from __future__ import annotations

import importlib.util
import os
import sys
from pathlib import Path

import torch

# ELF_B200_BOUNDS_CHECK=1 selects the debug variant (built with `python -m elf_b200.csrc.build --bounds-check`), whose
# tiled TMA copies validate their coordinates on the device and record a violation in the status word
_CHECKED = os.environ.get("ELF_B200_BOUNDS_CHECK", "0") not in ("", "0")
_BUILD_DIR = Path(__file__).resolve().parent.parent / "csrc" / ("_build_check" if _CHECKED else "_build")
_NAME = "elf_b200_C_check" if _CHECKED else "elf_b200_C"
_module = None
_load_error: Exception | None = None


def _try_load():
    global _module, _load_error
    if _module is not None or _load_error is not None:
        return
    so = _BUILD_DIR / f"{_NAME}.so"
    if not so.exists():
        _load_error = FileNotFoundError(f"{so} not found; run `python -m elf_b200.csrc.build{' --bounds-check' if _CHECKED else ''}`")
        return
    try:
        spec = importlib.util.spec_from_file_location(_NAME, so)
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)
        sys.modules[_NAME] = mod
        _module = mod
    except Exception as exc:  # missing libcuda on a CPU box, ABI mismatch, ...
        _load_error = exc


def available() -> bool:
    """True when the extension is loaded (it loads on CPU-only machines too; its CUDA
    entry points need a device, its host runtime does not)."""
    _try_load()
    return _module is not None


# Kernel launches per Python-visible entry point (a `gemm` call is one launch,
# `rmsnorm_bwd` two, ...), kept so that benchmarks can report how many of this package's
# kernels ran inside a timed region.
_LAUNCHES_PER_CALL = {
    "gemm": 1, "rmsnorm_fwd": 1, "rmsnorm_bwd": 3, "rope_": 1, "swiglu_fwd": 1, "swiglu_bwd": 1, "ce_fwd": 1,
    "ce_bwd": 1, "embedding_fwd": 1, "residual_add": 1, "pack_qkv_grad": 1, "ce_chunk_stats": 1, "ce_chunk_grad": 1, "embedding_bwd": 1, "embedding_bwd_sorted": 1, "adamw": 1, "scale_": 1, "attention_fwd": 1,
    "attention_bwd": 3, "push_reduce": 1, "push_ranges": 1, "finalize_reduce": 1, "p2p_signal": 1, "p2p_wait": 1, "gemm_dw_reduce": 1,
}
launch_count = 0


class _Counting:
    """Attribute proxy over the extension module that counts kernel launches."""

    def __init__(self, mod):
        object.__setattr__(self, "_mod", mod)
        object.__setattr__(self, "_cache", {})

    def __getattr__(self, name):
        cached = self._cache.get(name)
        if cached is not None:
            return cached
        fn = getattr(self._mod, name)
        n = _LAUNCHES_PER_CALL.get(name)
        if n is None or not callable(fn):
            return fn

        def counted(*args, __fn=fn, __n=n, **kwargs):
            global launch_count
            launch_count += __n
            return __fn(*args, **kwargs)

        self._cache[name] = counted
        return counted


_proxy = None


def get():
    """The extension module (behind a launch-counting proxy); raises with the reason when
    it cannot be loaded."""
    global _proxy
    _try_load()
    if _module is None:
        raise RuntimeError(f"elf_b200 native extension unavailable: {_load_error}")
    if _proxy is None:
        _proxy = _Counting(_module)
    return _proxy


def launches() -> int:
    """Kernels of this package launched so far in this process."""
    return launch_count


def cuda_ready() -> bool:
    return torch.cuda.is_available() and available()


def require_on_gpu() -> None:
    """Called by ops before they would fall back to torch: on a machine with a GPU a
    missing extension is an error, not a reason to run slowly."""
    if torch.cuda.is_available() and not available():
        raise RuntimeError(
            f"a CUDA device is present but the elf_b200 extension is not loaded ({_load_error}); "
            "build it with `python -m elf_b200.csrc.build`"
        )
