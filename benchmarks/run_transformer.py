#!/usr/bin/env python
"""Train a transformer through the pipeline and report throughput and memory.

Counterpart of the reference's ``benchmarks/run_transformer.py`` (same flags where they
make sense) with device-timed measurements:

    torchrun --nproc-per-node 8 benchmarks/run_transformer.py --architecture llama --model llama3-8b \
        --scheduler zbv --nmb 16 --mb-size 1 --niters 10
    torchrun --nproc-per-node 8 benchmarks/run_transformer.py --architecture llama --model llama-13b \
        --scheduler hanayo --dp 2 --nmb 16 --memory-budget 61440

``--architecture full|chain`` builds the GELU/LayerNorm zoo models and partitions them
automatically (``--partitioner``); ``--architecture llama`` builds only this rank's stages
directly on its GPU (the ``handcrafted`` partition of the reference).
"""

from __future__ import annotations

import argparse
import json
import logging
import os
import sys
import time

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import torch
import torch.distributed as dist

from benchmarks.benchmark_utils import ClockSampler, get_checkpointed_scheduler, get_offloaded_scheduler, init_dist, max_over_ranks, write_detailed_stats
from elf_b200 import Pipeline, PipelineConfig, Placement, replace_layer_with_layer_dw, sequential_signatures
from benchmarks.models.utils import add_transformer_args, model_config_from_args
from elf_b200.models.llama import LLAMA_CONFIGS, build_llama, build_llama_stages, llama_loss_fn
from elf_b200.models.simple import ChainTransformer, FullTransformer
from elf_b200.optim import DummyOptimizer, FusedAdamW, MixedPrecisionOptimizer
from elf_b200.registry import SCHEDULERS, TRACERS

logger = logging.getLogger("run_transformer")
_DTYPES = {"float16": torch.float16, "fp16": torch.float16, "bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32, "fp32": torch.float32}


def parse_args():
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    add_transformer_args(ap)  # --architecture, --name/--model, --config-file, dimensions, --dtype, --sdp-backend
    ap.add_argument("--batch-size", type=int, default=None, help="global batch per DP replica")
    ap.add_argument("--nmb", type=int, default=None)
    ap.add_argument("--mb-size", type=int, default=1)
    ap.add_argument("--opt-dtype", default=None, choices=sorted(_DTYPES))
    ap.add_argument("--opt-device", default="cuda", choices=["cpu", "cuda"])
    ap.add_argument("--no-optimizer", action="store_true")
    ap.add_argument("--partitioner", default="handcrafted", choices=["naive", "constrained", "metis", "dagP", "handcrafted"])
    ap.add_argument("--split-layers", action="store_true", help="llama: let stage boundaries fall between the attention half and the MLP half of a layer")
    ap.add_argument("--scheduler", default="1f1b", choices=["gpipe", "afab", "1f1b", "megatron", "hanayo", "zbh1", "zbh2", "zbv", "full_remat", "file", "auto"])
    ap.add_argument("--schedule-file")
    ap.add_argument("--interleaving", type=int, default=1)
    ap.add_argument("--dp", type=int, default=1)
    ap.add_argument("--niters", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--checkpointing", choices=["full", "simple", "selective"])
    ap.add_argument("--offloading", type=int)
    ap.add_argument("--prefetching-time", type=int, default=1)
    ap.add_argument("--log", choices=["none", "info", "debug"], default="info")
    ap.add_argument("--backend", default=None, choices=["nccl", "gloo", "mpi"])
    ap.add_argument("--stats-file")
    ap.add_argument("--profile", action="store_true")
    ap.add_argument("--memory-budget", type=int, help="MB per GPU; enables ILP rematerialisation")
    ap.add_argument("--tracer", default="default", choices=TRACERS.available() if len(TRACERS) else ["default"])
    ap.add_argument("--grad-sync", default="auto", choices=["auto", "nccl", "symm"])
    ap.add_argument("--check", action="store_true", help="before timing, compare one pipeline step (outputs, loss, every gradient) with the same model run in a single process")
    ap.add_argument("--p2p", default="auto", choices=["auto", "nccl", "copy"], help="stage-to-stage transport")
    ap.add_argument("--offload-ilp", action="store_true", help="with --memory-budget: let the ILP also offload activations to pinned host memory")
    return ap.parse_args()


def _with_zoo_api(model, loss_fn, sample, vocab):
    """Give a model that lacks them the ``get_sample`` / ``get_target`` / ``loss_fn`` members the
    correctness check calls (the Llama stages are plain ``nn.Sequential``)."""
    if hasattr(model, "get_sample"):
        return model
    shape = tuple(sample.shape[1:])

    def get_sample(n, dtype=None, device="cpu"):
        return torch.randint(0, vocab, (n, *shape), device=device)

    model.get_sample, model.get_target, model.loss_fn = get_sample, get_sample, loss_fn
    return model


def main():
    args = parse_args()
    if args.architecture is None and not args.config_file:
        args.architecture = "llama"  # this entry point's default; the option module's own default is "full"
    mcfg = model_config_from_args(args)
    args.architecture, args.model = mcfg["architecture"], mcfg["name"]
    local, rank, world = init_dist(args.backend)
    logging.basicConfig(level={"none": 100, "info": logging.INFO, "debug": logging.DEBUG}[args.log])
    device = torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else torch.device("cpu")
    dtype = mcfg["dtype"] if (args.dtype or args.config_file) else (torch.bfloat16 if device.type == "cuda" else torch.float32)
    pp = world // args.dp
    assert args.batch_size is not None or args.nmb is not None, "Batch size or number of micro-batches must be provided"
    batch = args.mb_size * args.nmb if args.batch_size is None else args.batch_size
    assert batch % args.mb_size == 0
    stored = None
    if args.scheduler == "file":
        with open(args.schedule_file) as f:
            stored = json.load(f)
        if "full_fwd" in stored:  # a stored ILP solution (benchmarks/plan_memory.py --out): its order plus its remat / offload tables
            from benchmarks.ilp_schedulers import RematScheduler

            scheduler = RematScheduler(stored)
        else:
            scheduler = SCHEDULERS["fixed"](stored)
    else:
        scheduler = args.scheduler
    if stored is not None and "placement" in stored:
        placement = Placement(stored["placement"])
    else:
        placement = Placement.default(args.scheduler, pp) * args.interleaving
    if args.checkpointing:
        scheduler = get_checkpointed_scheduler(scheduler, args.checkpointing)
    elif args.offloading:
        scheduler = get_offloaded_scheduler(scheduler, args.offloading, args.prefetching_time)

    t0 = time.time()
    pp_rank = rank % pp
    if args.architecture == "llama" and args.partitioner != "handcrafted":
        # graph front end on the Llama model: the worker rank builds the whole decoder as one flat
        # nn.Sequential of fused blocks, traces it, times every node on its GPU, cuts it with the
        # chosen partitioner and ships the stages; the other ranks only pass the sample
        cfg = LLAMA_CONFIGS[args.model]
        if args.seq_len:
            from dataclasses import replace as _replace

            cfg = _replace(cfg, seq_len=args.seq_len)
        model = build_llama(cfg, device=device, dtype=dtype, seed=1234, split_backward=True) if rank == 0 else None
        parts, signatures, partitioner = model, None, args.partitioner
        loss_fn, vocab, seq = llama_loss_fn, cfg.vocab, cfg.seq_len
        sample = torch.randint(0, vocab, (args.mb_size, seq), device=device)
        n_params = cfg.n_params()
    elif args.architecture == "llama":
        cfg = LLAMA_CONFIGS[args.model]
        mine = placement.get_ids(pp_rank)
        stages = build_llama_stages(cfg, len(placement), only=mine, device=device, dtype=dtype, seed=1234, placement=list(placement), split_layers=args.split_layers)
        if args.scheduler == "zbv" and pp > 1 and not args.checkpointing and not args.offloading and args.memory_budget is None:
            # ZB-V laid out for what the stages cost (layer halves per stage, LM head on the last one),
            # with the live-activation cap chosen by the timeline simulator
            import functools

            from elf_b200.models.llama import llama_stage_costs
            from elf_b200.scheduling.schedulers import generate_zbv_schedule

            scheduler = functools.partial(generate_zbv_schedule, cap="auto", cap_limit=6 * pp, ratios=(1.0, 1.4, 0.85),
                                          stage_costs=llama_stage_costs(cfg, len(placement), list(placement), args.split_layers))
        parts, signatures, partitioner = [stages[i] for i in mine], sequential_signatures(placement), False
        loss_fn, vocab, seq = llama_loss_fn, cfg.vocab, cfg.seq_len
        sample = torch.randint(0, vocab, (args.mb_size, seq), device=device)
        n_params = cfg.n_params()
    else:
        kw = {k: mcfg[k] for k in ("hidden_dim", "n_blocks", "seq_len", "num_heads", "num_kv_heads", "ffn_dim", "dropout", "sdp_backend")}
        if args.architecture == "full":
            kw["input_dim"] = mcfg["input_dim"]
        cls = FullTransformer if args.architecture == "full" else ChainTransformer
        model = cls(**kw).to(dtype)
        replace_layer_with_layer_dw(model)
        loss_fn = cls.loss_fn
        sample = model.get_sample(args.mb_size, dtype, device)
        n_params = sum(p.numel() for p in model.parameters())
        vocab, seq = getattr(model, "vocab", 0), model.seq_len
        partitioner = "constrained" if args.partitioner == "handcrafted" else args.partitioner
        parts, signatures = (model.to(device) if rank == 0 else model), None
    if rank == 0:
        print(f"The model has {n_params / 1e9:.2f}B parameters")
    budget = args.memory_budget
    if budget is not None and not args.no_optimizer:
        budget -= n_params * torch.empty(0, dtype=dtype).element_size() / world / 2**20
    config = PipelineConfig(partitioner=partitioner, scheduler=scheduler, placement=list(placement), tracer=args.tracer, pp=pp, dp=args.dp,
                            memory_budget=budget, signatures=signatures, outputs="device" if args.check else "none", grad_sync=args.grad_sync, p2p=args.p2p,
                            offload=args.offload_ilp)
    pipe = Pipeline(parts, sample, config=config)
    if world > 1:
        dist.barrier()
    partition_time = time.time() - t0
    if args.check:
        if partitioner is False:
            raise SystemExit("--check needs the un-partitioned model: use an automatic partitioner (--partitioner constrained|naive|metis|dagP)")
        from benchmarks.benchmark_utils import check_correctness

        reference_model = model if rank == 0 else None
        if world > 1:  # every rank needs the module (for its sample/target/loss functions); rank 0 holds the real one
            box = [None]
            if rank == 0:
                import copy

                with torch.device("meta"):
                    skeleton = copy.deepcopy(model).to("meta")
                box = [skeleton]
            dist.broadcast_object_list(box, src=0)
            reference_model = model if rank == 0 else box[0]
        tol = 1e-3 if dtype == torch.float32 else 5e-2
        report = check_correctness(_with_zoo_api(reference_model, loss_fn, sample, vocab), pipe, atol=tol, rtol=tol, batch=max(2, pp) * args.mb_size)
        if report:
            print(f"correctness check passed: max abs differences {report}")

    params = list(pipe.parameters())
    if args.no_optimizer or not params:
        opt = DummyOptimizer()
    elif device.type == "cuda" and dtype == torch.bfloat16 and args.opt_device == "cuda" and args.opt_dtype in (None, "float32", "fp32"):
        opt = FusedAdamW(params, lr=1e-4, eps=1e-5)
    else:
        opt = MixedPrecisionOptimizer(torch.optim.AdamW, params, dtype, _DTYPES[args.opt_dtype] if args.opt_dtype else dtype, torch.device(args.opt_device if device.type == "cuda" else "cpu"), lr=1e-4, eps=1e-5)

    def make_batch():
        if args.architecture == "chain":
            x = torch.randn(batch, seq, mcfg["hidden_dim"], dtype=dtype, device=device)
            return x, x.clone()
        tok = torch.randint(0, vocab, (batch, seq + 1), device=device)
        return tok[:, :-1].contiguous(), tok[:, 1:].contiguous()

    for _ in range(args.warmup):
        x, y = make_batch()
        opt.zero_grad()
        pipe(x, y, loss_fn, split_size=args.mb_size)
    batches = [make_batch() for _ in range(args.niters)]
    if device.type == "cuda":
        torch.cuda.reset_peak_memory_stats()
        torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    if args.profile and device.type == "cuda":
        torch.cuda.cudart().cudaProfilerStart()
    wall0 = time.time()
    with ClockSampler(local) as clocks:
        if device.type == "cuda":
            ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            ev0.record()
        for x, y in batches:
            opt.zero_grad()
            pipe(x, y, loss_fn, split_size=args.mb_size, profile=args.profile)
            opt.step()
        if device.type == "cuda":
            ev1.record()
            torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
    wall = time.time() - wall0
    if args.profile and device.type == "cuda":
        torch.cuda.cudart().cudaProfilerStop()
    dev_s = max_over_ranks(ev0.elapsed_time(ev1) / 1e3, device) if device.type == "cuda" else wall
    peak = torch.cuda.max_memory_allocated() / 2**30 if device.type == "cuda" else 0.0
    print(f"Rank {rank} : peak memory {peak:.2f} GB")
    if args.stats_file:
        write_detailed_stats(args.stats_file, pipe.detailed_stats, rank, world)
    if rank == 0:
        tokens = args.dp * batch * args.niters * seq
        s = pipe.stats
        bubble = 100.0 * s.get("bubble", 0.0) / s["total"] if os.environ.get("ELF_TIMINGS") and s.get("total") else None
        print(json.dumps({
            "model_creation_and_partition_s": round(partition_time, 2),
            "s_per_iter_device": dev_s / args.niters,
            "s_per_iter_wall": wall / args.niters,
            "tokens_per_s": tokens / dev_s,
            "bubble_pct": bubble,
            "peak_gb_rank0": peak,
            "clocks": clocks.summary(),
        }))
    pipe.clear()
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
