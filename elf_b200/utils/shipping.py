"""Move ``nn.Module`` objects between ranks.

Behavioural counterpart of the reference's ``send_models`` / ``recv_models`` /
``broadcast_models`` (``elf/utils.py:327-507``): the module *skeleton* travels as a
pickle with every parameter and buffer replaced by a ``meta`` placeholder, and the
tensor payload travels through the tensor path of ``torch.distributed``.

Differences, all deliberate:

* the payload is coalesced into one flat buffer per dtype, so a stage costs a
  handful of messages instead of two per tensor;
* shapes/dtypes ride inside the pickled skeleton (the placeholders already carry
  them), so there is no per-tensor metadata message;
* ``broadcast_models`` uses the same skeleton + flat-buffer scheme with
  ``dist.broadcast`` rather than pickling full weights;
* everything is device-agnostic: the transport device is CUDA with NCCL and CPU
  with gloo.
"""

from __future__ import annotations

import contextlib
from collections import OrderedDict
from typing import Dict, List, Sequence, Tuple

import torch
import torch.distributed as dist
import torch.nn as nn

__all__ = ["send_models", "recv_models", "broadcast_models", "transport_device"]


def transport_device(group=None) -> torch.device:
    """Device tensors must live on for p2p/collectives of ``group``'s backend."""
    backend = dist.get_backend(group) if dist.is_initialized() else "gloo"
    if "nccl" in str(backend) and torch.cuda.is_available():
        return torch.device("cuda", torch.cuda.current_device())
    return torch.device("cpu")


def _owner(model: nn.Module, qualified: str) -> Tuple[nn.Module, str]:
    path, _, leaf = qualified.rpartition(".")
    return (model.get_submodule(path) if path else model), leaf


def _named_tensors(model: nn.Module) -> List[Tuple[str, str, torch.Tensor]]:
    """``(kind, qualified name, tensor)``; a tensor reachable under several names (a module
    used twice) is listed once - the pickled skeleton keeps the sharing."""
    out = [("param", n, p) for n, p in model.named_parameters()]
    out += [("buffer", n, b) for n, b in model.named_buffers()]
    return out


@contextlib.contextmanager
def _as_skeleton(model: nn.Module):
    """Temporarily swap every parameter/buffer for a ``meta`` tensor of the same
    shape/dtype so that pickling the module ships structure only."""
    undo = []
    try:
        for kind, name, t in _named_tensors(model):
            mod, leaf = _owner(model, name)
            table = mod._parameters if kind == "param" else mod._buffers
            undo.append((table, leaf, table[leaf]))
            ghost = torch.empty_like(t, device="meta")
            table[leaf] = nn.Parameter(ghost, requires_grad=t.requires_grad) if kind == "param" else ghost
        yield model
    finally:
        for table, leaf, original in reversed(undo):
            table[leaf] = original


def _flatten_by_dtype(tensors: Sequence[torch.Tensor], device) -> "OrderedDict[torch.dtype, torch.Tensor]":
    groups: Dict[torch.dtype, List[torch.Tensor]] = OrderedDict()
    for t in tensors:
        groups.setdefault(t.dtype, []).append(t.detach().reshape(-1))
    flat = OrderedDict()
    for dt, parts in groups.items():
        flat[dt] = torch.cat([p.to(device) for p in parts]) if parts else torch.empty(0, dtype=dt, device=device)
    return flat


def _materialise(model: nn.Module, flats: Dict[torch.dtype, torch.Tensor], device) -> None:
    """Replace the ``meta`` placeholders of a received skeleton by views cut from
    the per-dtype flat buffers (tensors registered under several names stay shared)."""
    cursor = {dt: 0 for dt in flats}
    for kind, name, ghost in _named_tensors(model):
        n = ghost.numel()
        dt = ghost.dtype
        chunk = flats[dt][cursor[dt] : cursor[dt] + n].view(ghost.shape).to(device).clone()
        cursor[dt] += n
        mod, leaf = _owner(model, name)
        if kind == "param":
            mod._parameters[leaf] = nn.Parameter(chunk, requires_grad=ghost.requires_grad)
        else:
            mod._buffers[leaf] = chunk


def _layout(model: nn.Module) -> "OrderedDict[torch.dtype, int]":
    sizes: Dict[torch.dtype, int] = OrderedDict()
    for _, _, t in _named_tensors(model):
        sizes[t.dtype] = sizes.get(t.dtype, 0) + t.numel()
    return sizes


def send_models(models: Sequence[nn.Module], dst: int, group=None) -> None:
    """Send ``models`` to global rank ``dst``."""
    assert dist.is_initialized(), "torch.distributed must be initialized before calling send_models"
    dev = transport_device(group)
    with contextlib.ExitStack() as stack:
        for m in models:
            stack.enter_context(_as_skeleton(m))
        dist.send_object_list(list(models), dst=dst, group=group)
    for m in models:
        for flat in _flatten_by_dtype([t for _, _, t in _named_tensors(m)], dev).values():
            if flat.numel():
                dist.send(flat, dst=dst, group=group)


def recv_models(models: list, src: int, group=None, device=None) -> None:
    """Fill ``models`` (a list of the right length) with modules sent by ``src``."""
    assert dist.is_initialized(), "torch.distributed must be initialized before calling recv_models"
    dev = transport_device(group)
    target = torch.device(device) if device is not None else dev
    skeletons = [None] * len(models)
    dist.recv_object_list(skeletons, src=src, group=group)
    for i, m in enumerate(skeletons):
        flats = {}
        for dt, n in _layout(m).items():
            flats[dt] = torch.empty(n, dtype=dt, device=dev)
            if n:
                dist.recv(flats[dt], src=src, group=group)
        _materialise(m, flats, target)
        models[i] = m


def broadcast_models(models: list, src: int, group=None, device=None) -> None:
    """Replicate ``models`` from global rank ``src`` to every rank of ``group``."""
    dev = transport_device(group)
    target = torch.device(device) if device is not None else dev
    me = dist.get_rank()
    if me == src:
        with contextlib.ExitStack() as stack:
            for m in models:
                stack.enter_context(_as_skeleton(m))
            dist.broadcast_object_list(list(models), src=src, group=group)
        for m in models:
            for flat in _flatten_by_dtype([t for _, _, t in _named_tensors(m)], dev).values():
                if flat.numel():
                    dist.broadcast(flat, src=src, group=group)
            m.to(target)
    else:
        skeletons = [None] * len(models)
        dist.broadcast_object_list(skeletons, src=src, group=group)
        for i, m in enumerate(skeletons):
            flats = {}
            for dt, n in _layout(m).items():
                flats[dt] = torch.empty(n, dtype=dt, device=dev)
                if n:
                    dist.broadcast(flats[dt], src=src, group=group)
            _materialise(m, flats, target)
            models[i] = m
