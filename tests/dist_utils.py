"""Spawn helpers for multi-process CPU (gloo) tests."""

import os
import socket
import traceback

import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _entry(rank, world, port, fn, args, errors):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["RANK"] = str(rank)
    os.environ["WORLD_SIZE"] = str(world)
    torch.set_num_threads(1)
    try:
        dist.init_process_group("gloo", rank=rank, world_size=world)
        fn(rank, world, *args)
        dist.barrier()
    except Exception:
        errors.put((rank, traceback.format_exc()))
        raise
    finally:
        if dist.is_initialized():
            dist.destroy_process_group()


def run_ranks(fn, world: int, *args, timeout: float = 240.0):
    """Run ``fn(rank, world, *args)`` on ``world`` gloo ranks; raise on the first failure."""
    ctx = mp.get_context("spawn")
    errors = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_entry, args=(r, world, port, fn, args, errors), daemon=True) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout)
    failed = []
    while not errors.empty():
        failed.append(errors.get())
    for p in procs:
        if p.is_alive():
            p.terminate()
            failed.append((-1, "rank timed out"))
    bad = [p.exitcode for p in procs if p.exitcode not in (0, None)]
    if failed or bad:
        raise AssertionError("distributed test failed:\n" + "\n".join(f"[rank {r}]\n{tb}" for r, tb in failed) + f"\nexit codes: {bad}")
