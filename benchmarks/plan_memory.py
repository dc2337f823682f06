"""Plan a memory-budgeted pipeline offline: which activations to recompute or offload, on the CPU.

``Pipeline(memory_budget=...)`` profiles every stage on its GPU and solves the ILP with the
measured numbers.  This script answers the same question before any GPU is used, from analytic
estimates of a Llama-style stage (FLOPs at a given sustained rate for the durations, the tensors
the single-node layers keep for the memory), so that a configuration can be sized first:

    python benchmarks/plan_memory.py --name llama-70b --pp 8 --nmb 32 --scheduler zbv --memory-budget-gb 170 --offload
    python benchmarks/plan_memory.py --name llama-13b --pp 4 --nmb 16 --scheduler hanayo --memory-budget-gb 60

It prints the size of the ILP, the solver time, the planned step, the peak per rank and how many
(stage, micro-batch) slots use each option; ``--out FILE`` writes the solution in the form
``benchmarks/ilp_schedulers.py`` replays (counterpart of the reference's offline ILP flow,
``benchmarks/ilp_schedulers.py`` + ``elf/scheduling/ilp.py:683-697``).  The estimates are
analytic: a measured profile on the target GPUs replaces them when the job runs.
"""

from __future__ import annotations

import argparse
import json
import os
import sys
import time

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from elf_b200.models.llama import LLAMA_CONFIGS, llama_stage_ranges  # noqa: E402
from elf_b200.models.llama_costs import analytic_cost_model  # noqa: E402
from elf_b200.registry import SCHEDULERS  # noqa: E402
from elf_b200.scheduling.ilp import solve_remat  # noqa: E402
from elf_b200.utils.placement import Placement  # noqa: E402

MB = float(1 << 20)


def stage_statistics(cfg, placement, mb_size: int, tflops: float, bytes_per_param: float, nvlink_gbs: float = 700.0):
    """One statistics entry per stage (the keys ``profile_all_stages`` produces), estimated.

    Durations: FLOPs of the stage's layer parts (and the head) at ``tflops`` sustained, split into
    F / B / W by the cost model's shares.  Memory (bf16 activations): what a single-node decoder
    layer keeps per token after its forward - x, qkv, attention output, x + attention, gate/up, and
    the four W-pass operands (both norms' outputs, attention output, SwiGLU output) - and after its
    input-gradient pass (the W-pass operands and the four output gradients).  ``bytes_per_param``
    covers weights, gradients and optimizer state (16 for bf16 + fp32 master, m, v): the ILP counts
    ``2 x Mparams`` as resident, so ``Mparams`` is set to half of that."""
    n_stages = len(placement)
    cm = analytic_cost_model(cfg)
    ranges, k, costs = llama_stage_ranges(cfg, n_stages, list(placement), True, cm)
    tokens = mb_size * cfg.seq_len
    d, f, qkv = cfg.d_model, cfg.ffn, (cfg.n_heads + 2 * cfg.n_kv_heads) * cfg.head_dim
    layer_flops = tokens * (2 * d * qkv + 2 * d * d + 6 * d * f) + 2 * tokens * cfg.seq_len * d  # forward, causal attention
    layer_ms = 3.0 * layer_flops / (tflops * 1e12) * 1e3  # forward + both backward passes
    layer_params = d * qkv + d * d + 3 * d * f + 2 * d
    kept_f = 2.0 * tokens * (5 * d + qkv + 3 * f) / MB  # per layer, after the forward
    operands_w = 2.0 * tokens * (3 * d + f) / MB  # inputs of the four projections
    grads_w = 2.0 * tokens * (2 * d + qkv + 2 * f) / MB  # their output gradients
    boundary = 2.0 * tokens * d / MB
    stats = []
    for s, (first, last) in enumerate(ranges):
        layers = (last - first) / k
        t = costs[s] * layer_ms
        params = layers * layer_params
        act, ba, bg = layers * kept_f, layers * operands_w, layers * grads_w
        if s == 0:
            params += cfg.vocab * d
        if s == n_stages - 1:
            params += cfg.vocab * d + d
            logits = 2.0 * tokens * cfg.vocab / MB
            act, ba, bg = act + logits + boundary, ba + boundary, bg + logits
        one_layer = kept_f  # transient working set of the layer in flight
        stats.append({
            "T": {"f": t * cm.fbw[0], "b": t * cm.fbw[1], "w": t * cm.fbw[2]},
            "M": {"f": act + 2 * boundary, "b": ba + bg, "w": 0.0},
            "Mpeak": {"f": act + 2 * boundary + one_layer, "b": bg + one_layer, "w": one_layer / 4},
            "Mpeak_ckpt": 2 * boundary + one_layer,
            "Mparams": params * bytes_per_param / 2.0 / MB,
            "Mba": ba,
            "Mbg": bg,
            "Minput": boundary,
            "Moutput": boundary,
            "Tcomm": boundary / 1024.0 / nvlink_gbs * 1e3,
            "forward_remat_options": [],
            "backward_remat_options": [],
        })
    return stats, [round((b - a) / k, 2) for a, b in ranges]


def main(argv=None) -> dict:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--name", default="llama-70b", choices=sorted(LLAMA_CONFIGS))
    ap.add_argument("--pp", type=int, default=8)
    ap.add_argument("--nmb", type=int, default=32)
    ap.add_argument("--mb-size", type=int, default=1)
    ap.add_argument("--scheduler", default="zbv")
    ap.add_argument("--memory-budget-gb", type=float, default=170.0)
    ap.add_argument("--offload", action="store_true", help="let the ILP park activations in pinned host memory")
    ap.add_argument("--pcie-gbs", type=float, default=50.0)
    ap.add_argument("--tflops", type=float, default=1100.0, help="sustained bf16 rate of a whole layer (measured on B200 for the 8B shape: about 1100)")
    ap.add_argument("--bytes-per-param", type=float, default=16.0, help="weights + gradients + optimizer state (bf16 + fp32 master, m, v = 16)")
    ap.add_argument("--time-limit", type=int, default=120)
    ap.add_argument("--out", default=None, help="write the solution (JSON) for benchmarks/ilp_schedulers.py")
    args = ap.parse_args(argv)

    cfg = LLAMA_CONFIGS[args.name]
    placement = list(Placement.default(args.scheduler, args.pp))
    stats, layers = stage_statistics(cfg, placement, args.mb_size, args.tflops, args.bytes_per_param)
    budget_mb = args.memory_budget_gb * 1024.0
    resident = [0.0] * args.pp
    for s, st in enumerate(stats):
        resident[placement[s]] += 2.0 * st["Mparams"]
    report = {
        "model": args.name, "pp": args.pp, "micro_batches": args.nmb, "scheduler": args.scheduler, "placement": placement,
        "layers_per_stage": layers, "memory_budget_gb": args.memory_budget_gb, "offload": bool(args.offload),
        "resident_gb_per_rank": [round(v / 1024.0, 1) for v in resident],
        "activations_gb_per_stage_and_micro_batch": [round(st["M"]["f"] / 1024.0, 2) for st in stats],
        "binaries": len(placement) * args.nmb * (5 if args.offload else 3),
    }
    t0 = time.time()
    try:
        sol = solve_remat(stats, placement, SCHEDULERS[args.scheduler], args.nmb, budget_mb, time_limit=args.time_limit, offload=args.offload, pcie_gbs=args.pcie_gbs)
    except RuntimeError as exc:
        report.update(solver_s=round(time.time() - t0, 1), infeasible=str(exc))
        print(json.dumps(report))
        return report
    free = None
    try:
        free = solve_remat(stats, placement, SCHEDULERS[args.scheduler], args.nmb, 1e12, time_limit=args.time_limit)
    except RuntimeError:
        pass
    count = lambda name: int(sum(map(sum, sol.get(name, [])))) if name in sol else 0
    report.update(
        solver_s=round(time.time() - t0, 1),
        planned_step_ms=round(sol["objective"], 1),
        unconstrained_step_ms=round(free["objective"], 1) if free else None,
        unconstrained_peak_gb=round(max(free["peak_mems"]) / 1024.0, 1) if free else None,
        peak_gb_per_rank=[round(v / 1024.0, 1) for v in sol["peak_mems"]],
        slots={"total": len(placement) * args.nmb, "full_fwd": count("full_fwd"), "offload": count("offload"), "activations_bwd": count("activations_bwd"), "full_bwd": count("full_bwd")},
    )
    if args.out:
        with open(args.out, "w") as fh:
            json.dump(sol, fh)
    print(json.dumps(report))
    return report


if __name__ == "__main__":
    main()
