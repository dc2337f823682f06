#!/usr/bin/env python
"""Headline benchmark: training throughput of a Llama-3-8B-shaped decoder under a
Zero-Bubble-V pipeline schedule (bf16, 16 micro-batches of one 4096-token sequence).

    python bench.py --gpus 1 --steps 5 --warmup 3
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
        --master-port 29511 bench.py --gpus 8 --steps 5 --warmup 3
    python bench.py --impl reference ...      # the unmodified reference package, same config

One rank per GPU; pp = number of GPUs, dp = 1 (strong scaling: the model and the global
batch are fixed, stages get thinner as GPUs are added).  Rank 0 prints ONE JSON line.
``value`` is device-timed (CUDA events, max over ranks) with inputs already on the device;
``e2e`` repeats the measurement through the same public API with each step's token ids
copied from pinned host memory and the loss read back to the host.
"""

from __future__ import annotations

import argparse
import json
import os
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

BASELINE_TOKENS_PER_S = None  # the reference publishes no number for this configuration


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=4)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--model", default="llama3-8b")
    ap.add_argument("--scheduler", default="zbv")
    ap.add_argument("--nmb", type=int, default=16)
    ap.add_argument("--mb-size", type=int, default=1)
    ap.add_argument("--seq-len", type=int, default=None)
    ap.add_argument("--layers", type=int, default=None, help="override the layer count (debugging only; the result is then not the headline number)")
    ap.add_argument("--dp", type=int, default=1)
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--whole-layers", action="store_true", help="cut stages at layer boundaries only (for comparison)")
    ap.add_argument("--split-halves", action="store_true", help="cut stages between attention and MLP halves only (default: thirds when they balance the ranks better)")
    ap.add_argument("--split-thirds", action="store_true", help="also allow a stage boundary after the MLP's SwiGLU (two tensors cross it); finer balance for deep pipelines")
    ap.add_argument("--timeline", default=None, help="write every rank's per-operation device timeline of one extra step (JSON) to this file")
    ap.add_argument("--chunked-head", action="store_true", help="LM head + cross entropy with the vocabulary in chunks: the logits (1 GB per micro-batch) are never materialised, at the price of one more pass over the head's matrix")
    ap.add_argument("--grad-sync", choices=["auto", "nccl", "symm"], default="auto", help="with --dp > 1: peer-memory gradient exchange fused into the weight-gradient GEMM, or NCCL all-reduce")
    ap.add_argument("--p2p", choices=["auto", "nccl", "copy"], default="auto", help="stage-to-stage transport: NCCL send/recv kernels, or copy-engine writes into the consumer's ring buffer")
    ap.add_argument("--no-calibrate", action="store_true", help="cut the stages and lay the schedule out for the built-in cost constants instead of times measured at start-up (for comparison)")
    return ap.parse_args()


def run_ours(args):
    import torch
    import torch.distributed as dist

    from benchmarks.benchmark_utils import ClockSampler, init_dist, max_over_ranks
    from elf_b200 import Pipeline, Placement
    from elf_b200.models.llama import LLAMA_CONFIGS, build_llama_stages, choose_llama_cut, llama_loss_fn, llama_stage_costs, llama_stage_ranges, llama_stage_signatures
    from elf_b200.ops import _ext
    from elf_b200.optim import DummyOptimizer, FusedAdamW
    from dataclasses import replace

    local, rank, world = init_dist()
    assert world == args.gpus, f"--gpus {args.gpus} but WORLD_SIZE={world}; launch with torch.distributed.run"
    device = torch.device("cuda", torch.cuda.current_device())
    cfg = LLAMA_CONFIGS[args.model]
    if args.seq_len:
        cfg = replace(cfg, seq_len=args.seq_len)
    if args.layers:
        cfg = replace(cfg, n_layers=args.layers)
    dp = args.dp
    pp = world // dp
    placement = Placement.default(args.scheduler, pp)
    pp_rank = rank % pp
    mine = placement.get_ids(pp_rank)
    # stage boundaries may fall between the attention half and the MLP half of a layer: whole
    # layers cannot balance 32 layers + the LM head (2.2 layers' worth) over 8 ranks
    # what an attention half, the two MLP parts, the embedding and the head + loss cost on this GPU,
    # timed before the model is built (a second or two): the cut balances measured time per rank
    cost_model = None
    if pp > 1 and not args.no_calibrate and not args.whole_layers:
        from elf_b200.models.llama_costs import measure_cost_model

        cost_model = measure_cost_model(cfg, device, mb_size=args.mb_size)
        cost_model.micro_batches = args.nmb  # lets the cut allow for the pipeline's fill (deep ranks start late once per step)
    if pp == 1 or args.whole_layers:
        split_layers = False
    elif args.split_thirds:
        split_layers = "thirds"
    elif args.split_halves or cost_model is None:
        split_layers = True
    else:
        split_layers = choose_llama_cut(cfg, len(placement), list(placement), cost_model)
    cut = dict(placement=list(placement), split_layers=split_layers, cost_model=cost_model)
    stages = build_llama_stages(cfg, len(placement), only=mine, device=device, seed=1234, fused_head_loss=args.chunked_head, **cut)
    parts = [stages[i] for i in mine]
    stage_costs = llama_stage_costs(cfg, len(placement), **cut)
    signatures = llama_stage_signatures(cfg, len(placement), **cut)
    ranges, parts_per_layer, _ = llama_stage_ranges(cfg, len(placement), **cut)
    counts = [round((b - a) / parts_per_layer, 2) for a, b in ranges]
    scheduler, sched_note = args.scheduler, args.scheduler
    if args.scheduler == "zbv" and pp > 1:
        # ZB-V laid out for what the stages cost: layer counts differ per stage, the last stage
        # also runs the LM head, and B is longer than F and W (attention backward).  Up to 6p
        # live (stage, micro-batch) activations per rank instead of 2p: memory is not scarce here.
        import functools

        from elf_b200.scheduling.schedulers import generate_zbv_schedule

        ratios = tuple(round(v / cost_model.fbw[0], 3) for v in cost_model.fbw) if cost_model is not None else (1.0, 1.25, 0.9)
        scheduler = functools.partial(generate_zbv_schedule, cap="auto", cap_limit=6 * pp, stage_costs=stage_costs, ratios=ratios)
        sched_note = f"zbv (list-scheduled with per-stage costs, F:B:W = {ratios[0]}:{ratios[1]}:{ratios[2]}, live-activation cap per rank chosen in [2p, 6p] by the timeline simulator)"
    pipe = Pipeline(parts, None, partitioner=False, scheduler=scheduler, placement=list(placement), dp=dp, outputs="none", signatures=signatures, p2p=args.p2p, grad_sync=args.grad_sync)
    params = list(pipe.parameters())
    opt = FusedAdamW(params, lr=1e-4, betas=(0.9, 0.95), eps=1e-5, weight_decay=0.1) if params else DummyOptimizer()

    batch = args.nmb * args.mb_size
    n_batches = args.warmup + 2 * args.steps + 1
    gen = torch.Generator().manual_seed(1000 + rank // pp)
    host = [torch.randint(0, cfg.vocab, (batch, cfg.seq_len + 1), generator=gen).pin_memory() for _ in range(n_batches)]

    def to_device(tok):
        tok = tok.to(device, non_blocking=True)
        return tok[:, :-1].contiguous(), tok[:, 1:].contiguous()

    loss_fn = llama_loss_fn
    if args.chunked_head and stages[-1] is not None:
        from elf_b200.ops.head_loss import ChunkedHeadLoss

        loss_fn = ChunkedHeadLoss(stages[-1][-1])

    def step(ids, tgt):
        opt.zero_grad()
        _, loss = pipe(ids, tgt, loss_fn, split_size=args.mb_size)
        opt.step()
        return loss

    def fence():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    it = iter(host)
    calibrated = None
    for w in range(args.warmup):
        timed_step = scheduler is not args.scheduler and not args.no_calibrate and w == min(1, args.warmup - 2) and args.warmup >= 2
        if timed_step:
            os.environ["ELF_TIMINGS"] = "1"
        try:
            loss = step(*to_device(next(it)))
        finally:
            os.environ.pop("ELF_TIMINGS", None)
        if timed_step:
            # profile-guided schedule: lay ZB-V out again for the measured F / B / W time of every
            # stage (the analytic stage costs above are only the starting point); the remaining
            # warm-up steps and everything timed run the re-laid schedule
            calibrated = pipe.measured_stage_costs()
            # robust: the durations drift by a percent or two per rank over the following steps; keep a layout that stays short when they do
            pipe.set_scheduler(functools.partial(generate_zbv_schedule, cap="auto", cap_limit=6 * pp, stage_costs=calibrated, robust=0.02))
            sched_note = "zbv (list-scheduled for the F / B / W time of every stage measured in a warm-up step, live-activation cap per rank chosen in [2p, 6p] by the timeline simulator over perturbed copies of those times)"
    # ---- device-timed region: inputs resident on the device -------------------------
    resident = [to_device(next(it)) for _ in range(args.steps)]
    fence()
    torch.cuda.reset_peak_memory_stats()
    launches0 = _ext.launches()
    with ClockSampler(local) as clocks:
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        for ids, tgt in resident:
            loss = step(ids, tgt)
        end.record()
        fence()
    dev_ms = max_over_ranks(start.elapsed_time(end), device)
    from elf_b200.ops import gemm as _gemm

    _gemm.check_status(device)  # a kernel that gave up on a bounded wait must not pass as a fast step
    launches = _ext.launches() - launches0
    stats = dict(pipe.stats)
    peak_gb = max_over_ranks(torch.cuda.max_memory_allocated() / 2**30, device)
    last_loss = float(loss.item()) if loss is not None else None
    del resident
    # ---- end-to-end region: H2D of the step's tokens, D2H of its loss ---------------
    e2e = None
    if not args.no_e2e:
        fence()
        t0 = time.perf_counter()
        start.record()
        for _ in range(args.steps):
            tok = next(it)
            loss = step(*to_device(tok))
            if loss is not None:
                last_loss = float(loss.item())  # device -> host read of the step's result
        end.record()
        fence()
        e2e_ms = max_over_ranks(start.elapsed_time(end), device)
        tokens = dp * batch * cfg.seq_len * args.steps
        owns_io = pipe.is_first() or pipe.is_last()
        e2e = {
            "value": tokens / (e2e_ms / 1e3),
            "unit": "tokens/s",
            "ms_per_step": e2e_ms / args.steps,
            "h2d_bytes_per_step": int(host[0].numel() * host[0].element_size()) if owns_io else 0,
            "d2h_bytes_per_step": 4 if pipe.is_last() else 0,
            "wall_ms_per_step": (time.perf_counter() - t0) * 1e3 / args.steps,
        }
    # ---- one more step, outside every timed region, with per-operation timers: bubble share ----
    bubble = None
    os.environ["ELF_TIMINGS"] = "1"
    try:
        fence()
        step(*to_device(next(it)))
        fence()
        st = pipe.stats
        mine_pct = 100.0 * st["idle"] / st["total"] if st.get("total") else 0.0
        # mean duration of F / B / W per stage hosted here, from the per-operation timers
        import re

        per_stage = {}
        for name, secs in pipe.detailed_stats["all_events"].items():
            m = re.match(r"(forward|backward_inputs|backward_params)\((\d+):\d+\)", name)
            if m:
                per_stage.setdefault(int(m.group(2)), {}).setdefault(m.group(1), []).append(secs * 1e3)
        mine_ops = {s: [round(sum(v.get(k, [0.0])) / max(1, len(v.get(k, [0.0]))), 3) for k in ("forward", "backward_inputs", "backward_params")] for s, v in per_stage.items()}
        every = [None] * world
        mine_tl = {"timeline": pipe.detailed_stats.get("timeline", {}), "host_enqueue": pipe.detailed_stats.get("host_enqueue", {}), "total_s": st.get("total")}
        if world > 1:
            dist.all_gather_object(every, (mine_pct, mine_ops, mine_tl if args.timeline else None))
        else:
            every = [(mine_pct, mine_ops, mine_tl if args.timeline else None)]
        op_ms = {}
        for _, ops, _tl in every:
            op_ms.update(ops)
        if args.timeline and rank == 0:
            os.makedirs(os.path.dirname(os.path.abspath(args.timeline)), exist_ok=True)
            with open(args.timeline, "w") as f:
                json.dump({"placement": list(placement), "nmb": args.nmb, "pp": pp, "dp": dp, "ranks": {str(r): tl for r, (_, _, tl) in enumerate(every)}}, f)
        every = [p for p, _, _tl in every]
        bubble = {
            "bubble_pct_mean": sum(every) / world,
            "bubble_pct_max": max(every),
            "per_rank": [round(v, 2) for v in every],
            "stage_op_ms_f_b_w": {str(k): op_ms[k] for k in sorted(op_ms)},
            "stage_costs_analytic": [round(c, 2) for c in stage_costs],
            "stage_ms_calibrated_f_b_w": [[round(1e3 * v, 3) for v in t] for t in calibrated] if calibrated else None,
            "note": "one extra step with per-operation CUDA-event timers: share of the step in which a rank runs no forward / backward / loss / optimizer-free compute operation (waiting for peers, p2p, launch gaps)",
        }
    finally:
        os.environ.pop("ELF_TIMINGS", None)
    tokens = dp * batch * cfg.seq_len * args.steps
    value = tokens / (dev_ms / 1e3)
    line = {
        "metric": "training throughput, tokens/sec (device-timed, max over ranks)",
        "impl": "ours",
        "value": value,
        "unit": "tokens/s",
        "n_gpus": world,
        "steps": args.steps,
        "warmup": args.warmup,
        "ms_per_step": dev_ms / args.steps,
        "higher_is_better": True,
        "scaling": "strong",
        "vs_baseline": (value / BASELINE_TOKENS_PER_S) if BASELINE_TOKENS_PER_S else None,
        "dtype": "bf16",
        "data": "synthetic uniform token ids, N(0,0.02) random-init weights",
        "config": {
            "model": f"{args.model} ({cfg.n_layers} layers, d={cfg.d_model}, {cfg.n_heads}q/{cfg.n_kv_heads}kv heads, ffn={cfg.ffn}, vocab={cfg.vocab})",
            "global_batch": dp * batch,
            "micro_batches": args.nmb,
            "micro_batch_size": args.mb_size,
            "seq_len": cfg.seq_len,
            "parallelism": f"pp{pp}" + (f"xdp{dp}" if dp > 1 else ""),
            "scheduler": sched_note,
            "placement": list(placement),
            "layers_per_stage": counts,
            "stage_cut": {"split_layers": split_layers, "cost_model": ({k: (round(v, 4) if isinstance(v, float) else v) for k, v in cost_model.to_dict().items()} if cost_model else "built-in constants")},
            "optimizer": "fused AdamW, fp32 master/m/v, step inside the timed region",
            "lm_head": "vocabulary-chunked head + cross entropy (no logits tensor)" if args.chunked_head else "head GEMM + cross-entropy kernels over bf16 logits",
            "p2p": (pipe.channels.transport if pipe.channels is not None else "none"),
            "grad_sync": ("none" if dp == 1 else ("symm (peer-memory push from the weight-gradient GEMM epilogue)" if pipe.grad_sync is not None else "nccl all-reduce")),
            "l2": "working set (weights + activations, tens of GB) far exceeds the 126 MB L2; no flush needed",
        },
        "clocks": clocks.summary(),
        "e2e": e2e,
        "gpu_launches": launches,
        "bubble": bubble,
        "peak_gb_per_gpu": peak_gb,
        "loss": last_loss,
        "host_stats_last_step": {k: round(v, 6) for k, v in stats.items()},
    }
    pipe.clear()
    if rank == 0:
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def main():
    args = parse_args()
    dump_after = os.environ.get("ELF_B200_DUMP_STACKS_AFTER")
    if dump_after:  # debugging aid: write every thread's Python stack to a file after so many seconds, then exit
        import faulthandler

        path = os.path.join(os.environ.get("ELF_B200_DUMP_DIR", "."), f"stacks_rank{os.environ.get('RANK', '0')}.txt")
        main._stack_file = open(path, "w")
        faulthandler.dump_traceback_later(float(dump_after), exit=True, file=main._stack_file)
    if args.impl == "reference":
        from baseline.reference_arm import run_reference

        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
