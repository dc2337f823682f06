#!/usr/bin/env python
"""Roofline of the fused weight-gradient GEMM + data-parallel gradient push.

    python -m torch.distributed.run --nproc-per-node 2 --master-addr 127.0.0.1 benchmarks/dp_fused_roofline.py

For the matrices of one Llama-3-8B decoder layer (M = 4096 tokens) each rank times, with CUDA
events after warm-up, max over ranks:
  gemm        dW += dY^T X                       (tcgen05 kernel, local store only)
  fused       the same launch whose epilogue also stores every tile into the peer's inbox
              and whose last CTA raises the peer's flag
  finalize    grad = scale * (local + inbox)     (local reads only)
  nccl        all_reduce of the gradient matrix  (what the unfused path would add)
and reports fused time against its roofline: the slower of FLOPs / measured GEMM peak and
bytes-over-NVLink / measured peer-copy bandwidth.
"""

import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from elf_b200.ops import _ext, gemm as G  # noqa: E402
from elf_b200.parallel.symm import SymmetricBuffer  # noqa: E402

GEMM_PEAK_TFLOPS = 1381.9  # cuBLAS bf16, sustained, measured on this pool
NVLINK_GBS = 770.0         # peer copy, per direction, measured on this pool


def timed(fn, iters=20, warm=3):
    for _ in range(warm):
        fn()
    torch.cuda.synchronize()
    dist.barrier()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(iters):
        fn()
    b.record()
    torch.cuda.synchronize()
    t = torch.tensor([a.elapsed_time(b) / iters], device="cuda", dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
    dev = torch.device("cuda", torch.cuda.current_device())
    dist.init_process_group("nccl", device_id=dev)
    group = dist.group.WORLD
    peers = [p for p in range(world) if p != rank]
    slot_on = {p: (rank if rank < p else rank - 1) for p in peers}
    M = 4096
    rows = []
    for name, n_out, n_in in [("wqkv", 6144, 4096), ("wo", 4096, 4096), ("w_gate_up", 28672, 4096), ("w_down", 4096, 14336)]:
        numel = n_out * n_in
        dy = torch.randn(M, n_out, device=dev, dtype=torch.bfloat16)
        x = torch.randn(M, n_in, device=dev, dtype=torch.bfloat16)
        grad = torch.zeros(n_out, n_in, device=dev, dtype=torch.bfloat16)
        inbox = SymmetricBuffer.allocate((world - 1) * numel, torch.bfloat16, group, dev)
        flags = SymmetricBuffer.allocate(world - 1, torch.int32, group, dev)
        counter = torch.zeros(1, dtype=torch.int32, device=dev)
        epoch = [0]

        def plain():
            G.linear_weight_grad(dy, x, out=grad)

        def fused():
            epoch[0] += 1
            push = {
                "push_out": [inbox.peer_address(p, slot_on[p] * numel * 2) for p in peers],
                "push_flags": [flags.peer_address(p, slot_on[p] * 4) for p in peers],
                "push_flag_value": epoch[0],
                "push_counter": counter,
            }
            G.linear_weight_grad(dy, x, out=grad, push=push)

        wait = torch.zeros(1, dtype=torch.int32, device=dev)

        def finalize():
            _ext.get().finalize_reduce(grad.view(-1), inbox.local, world - 1, flags.local, 1, wait, epoch[0], 0.5, 5000.0, G.status(dev))

        t_plain = timed(plain)
        t_fused = timed(fused)
        dist.barrier()
        t_final = timed(finalize)
        t_nccl = timed(lambda: dist.all_reduce(grad, op=dist.ReduceOp.AVG))
        torch.cuda.synchronize()
        G.check_status(dev)
        flops = 2.0 * M * n_out * n_in
        t_compute = flops / (GEMM_PEAK_TFLOPS * 1e12) * 1e3
        t_link = (world - 1) * numel * 2 / (NVLINK_GBS * 1e9) * 1e3
        roof = max(t_compute, t_link)
        rows.append({
            "matrix": name, "shape": [n_out, n_in], "gemm_ms": round(t_plain, 4), "fused_gemm_push_ms": round(t_fused, 4),
            "finalize_ms": round(t_final, 4), "nccl_allreduce_ms": round(t_nccl, 4), "roofline_ms": round(roof, 4),
            "roofline_bound": "compute" if t_compute >= t_link else "nvlink", "fused_fraction_of_roofline": round(roof / t_fused, 3),
            "fused_tflops": round(flops / t_fused / 1e9, 1), "push_gbs": round((world - 1) * numel * 2 / t_fused / 1e6, 1),
            "unfused_total_ms": round(t_plain + t_nccl, 4), "fused_total_ms": round(t_fused + t_final, 4),
        })
        del inbox, flags
    if rank == 0:
        print(json.dumps({"world": world, "tokens": M, "gemm_peak_tflops": GEMM_PEAK_TFLOPS, "nvlink_gbs": NVLINK_GBS, "rows": rows}, indent=1))
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
