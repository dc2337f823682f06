#!/usr/bin/env python
"""How much does stage-to-stage traffic slow the compute it overlaps with?

Two ranks (one per GPU) each run a loop of weight-gradient-sized GEMMs of this package on
their compute stream while activation-sized messages (32 MiB by default) cross NVLink in
both directions on side streams, through

* ``nccl``  ``isend`` / ``irecv`` on a dedicated 2-rank communicator per direction (what the
            pipeline's channels do): the transfers are kernels that need SMs on both GPUs;
* ``ce``    a copy-engine copy into the peer's buffer in symmetric memory: no SMs involved.

Printed per mode: milliseconds per GEMM (CUDA events on the compute stream, max over the two
ranks), the slow-down against the loop without traffic, and the time a message takes when
nothing else runs.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 \
        --master-port 29533 benchmarks/p2p_overlap.py
"""

from __future__ import annotations

import argparse
import json
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def main():
    import torch
    import torch.distributed as dist

    from benchmarks.benchmark_utils import init_dist, max_over_ranks
    from elf_b200.ops import gemm

    ap = argparse.ArgumentParser()
    ap.add_argument("--iters", type=int, default=40)
    ap.add_argument("--msg-mib", type=int, default=32)
    ap.add_argument("--m", type=int, default=4096)
    ap.add_argument("--n", type=int, default=14336)
    ap.add_argument("--k", type=int, default=4096)
    ap.add_argument("--msgs-per-gemm", type=int, default=1)
    args = ap.parse_args()

    local, rank, world = init_dist()
    assert world == 2, "run on exactly two ranks"
    dev = torch.device("cuda", torch.cuda.current_device())
    peer = 1 - rank
    g_fwd = dist.new_group([0, 1])
    g_bwd = dist.new_group([0, 1])

    x = torch.randn(args.m, args.k, device=dev, dtype=torch.bfloat16)
    w = torch.randn(args.n, args.k, device=dev, dtype=torch.bfloat16)
    numel = args.msg_mib * (1 << 20) // 2
    out_msg = torch.randn(numel, device=dev, dtype=torch.bfloat16)
    in_msg = torch.empty_like(out_msg)

    import torch.distributed._symmetric_memory as symm_mem

    inbox = symm_mem.empty(numel, dtype=torch.bfloat16, device=dev)
    handle = symm_mem.rendezvous(inbox, group=dist.group.WORLD.group_name)
    peer_inbox = handle.get_buffer(peer, (numel,), torch.bfloat16)
    side = torch.cuda.Stream(dev)

    def fence():
        torch.cuda.synchronize()
        dist.barrier()
        torch.cuda.synchronize()

    def traffic_nccl():
        works = []
        for _ in range(args.msgs_per_gemm):
            # rank 0 sends "forward" and receives "backward"; rank 1 the other way round
            if rank == 0:
                works.append(dist.isend(out_msg, dst=1, group=g_fwd))
                works.append(dist.irecv(in_msg, src=1, group=g_bwd))
            else:
                works.append(dist.irecv(in_msg, src=0, group=g_fwd))
                works.append(dist.isend(out_msg, dst=0, group=g_bwd))
        return works

    def traffic_ce():
        with torch.cuda.stream(side):
            for _ in range(args.msgs_per_gemm):
                peer_inbox.copy_(out_msg, non_blocking=True)
        return []

    def run(mode):
        keep = []
        fence()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(args.iters):
            if mode == "nccl":
                keep.extend(traffic_nccl())
            elif mode == "ce":
                traffic_ce()
            gemm.matmul_nt(x, w)
        b.record()
        for wk in keep:
            wk.wait()
        fence()
        return max_over_ranks(a.elapsed_time(b), dev) / args.iters

    def message_alone(mode):
        fence()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        keep = []
        a.record()
        for _ in range(args.iters):
            if mode == "nccl":
                for wk in traffic_nccl():
                    wk.wait()
            else:
                traffic_ce()
                torch.cuda.current_stream().wait_stream(side)
        b.record()
        fence()
        del keep
        return max_over_ranks(a.elapsed_time(b), dev) / args.iters / args.msgs_per_gemm

    # warm-up: communicators, kernels, clocks
    for mode in ("none", "nccl", "ce"):
        run(mode)
    res = {}
    for mode in ("none", "nccl", "ce", "none", "nccl", "ce"):
        res.setdefault(mode, []).append(run(mode))
    alone = {m: message_alone(m) for m in ("nccl", "ce")}
    gemm.check_status(dev)
    if rank == 0:
        base = min(res["none"])
        out = {
            "gemm": [args.m, args.n, args.k],
            "message_mib": args.msg_mib,
            "messages_per_gemm_each_way": args.msgs_per_gemm,
            "ms_per_gemm": {k: [round(v, 4) for v in vs] for k, vs in res.items()},
            "slowdown_vs_no_traffic": {k: round(min(vs) / base, 4) for k, vs in res.items()},
            "message_alone_ms": {k: round(v, 4) for k, v in alone.items()},
            "nccl_env": {k: v for k, v in os.environ.items() if k.startswith("NCCL_")},
        }
        print(json.dumps(out), flush=True)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
