"""Worker for the multi-GPU tests (launched with torch.distributed.run, one rank per GPU).

    python -m torch.distributed.run --nproc-per-node N tests/multigpu_worker.py <case>

Cases
  dp_symm     pp=1, dp=N: gradients after a step with the peer-memory exchange equal those
              of the NCCL all-reduce path and of a single-process reference
  pp          pp=N, dp=1 ZB-V: loss and gradients equal the single-process reference
  pp_dp       pp=N/2, dp=2 1F1B with the peer-memory exchange
  pp_copy     pp=N ZB-V with stage-to-stage traffic on the copy-engine transport from the second
              step on (three steps; loss and gradients equal the single-process reference)
"""

import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from elf_b200 import Pipeline, Placement  # noqa: E402
from elf_b200.models.llama import LlamaConfig, build_llama_stages, llama_loss_fn  # noqa: E402
from elf_b200.ops import gemm  # noqa: E402


def rel(a, b):
    return ((a.float() - b.float()).norm() / b.float().norm().clamp_min(1e-12)).item()


def reference(cfg, n_stages, tokens, dev, **cut):
    """Whole model on this GPU with torch ops in fp32: loss and gradients per stage."""
    stages = build_llama_stages(cfg, n_stages, device=dev, dtype=torch.float32, seed=7, split_backward=False, **cut)
    bf16 = build_llama_stages(cfg, n_stages, device=dev, dtype=torch.bfloat16, seed=7, split_backward=False, **cut)
    for s32, s16 in zip(stages, bf16):  # same (bf16-rounded) weights as the pipeline
        s32.load_state_dict({k: v.float() for k, v in s16.state_dict().items()})
    gemm.set_enabled(False)
    try:
        x = tokens[:, :-1]
        for s in stages:
            x = s(x)
        loss = torch.nn.functional.cross_entropy(x.reshape(-1, x.size(-1)), tokens[:, 1:].reshape(-1))
        loss.backward()
    finally:
        gemm.set_enabled(True)
    return loss.detach(), [{n: p.grad for n, p in s.named_parameters()} for s in stages]


def run(case):
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
    dev = torch.device("cuda", torch.cuda.current_device())
    dist.init_process_group("nccl", device_id=dev)
    cfg = LlamaConfig(n_layers=4, d_model=256, n_heads=4, n_kv_heads=2, ffn=512, vocab=1024, seq_len=128, rope_theta=10000.0)
    if case == "dp_symm":
        pp, dp, sched, modes = 1, world, "zbh1", ["nccl", "symm"]
    elif case == "pp":
        pp, dp, sched, modes = world, 1, "zbv", ["nccl"]
    elif case == "pp_split":  # stage boundaries inside layers, ZB-V with the simulator-chosen activation cap
        pp, dp, sched, modes = world, 1, "zbv", ["nccl"]
        cfg = LlamaConfig(n_layers=5, d_model=256, n_heads=4, n_kv_heads=2, ffn=512, vocab=1024, seq_len=128, rope_theta=10000.0)
    elif case == "pp_dp":
        pp, dp, sched, modes = world // 2, 2, "1f1b", ["symm"]
    elif case == "pp_copy":
        pp, dp, sched, modes = world, 1, "zbv", ["nccl"]
    else:
        raise SystemExit(f"unknown case {case}")
    placement = Placement.default(sched, pp)
    n_stages = len(placement)
    per_replica, nmb = 4, 4
    gen = torch.Generator().manual_seed(3)
    tokens = torch.randint(0, cfg.vocab, (dp * per_replica, cfg.seq_len + 1), generator=gen).to(dev)
    cut = dict(placement=list(placement), split_layers=True) if case == "pp_split" else {}
    scheduler = sched
    if case == "pp_split":
        import functools

        from elf_b200.models.llama import llama_stage_costs
        from elf_b200.scheduling.schedulers import generate_zbv_schedule

        scheduler = functools.partial(generate_zbv_schedule, cap="auto", stage_costs=llama_stage_costs(cfg, n_stages, list(placement), True), ratios=(1.0, 1.25, 0.9))
    ref_loss, ref_grads = reference(cfg, n_stages, tokens, dev, **cut)
    pp_rank, dp_rank = rank % pp, rank // pp
    mine = placement.get_ids(pp_rank)
    results = {}
    for mode in modes:
        stages = build_llama_stages(cfg, n_stages, only=mine, device=dev, seed=7, **cut)
        pipe = Pipeline([stages[i] for i in mine], None, partitioner=False, scheduler=scheduler, placement=list(placement), dp=dp, outputs="none", grad_sync=mode,
                        p2p="copy" if case == "pp_copy" else "nccl")
        if mode == "symm":
            assert pipe.grad_sync is not None, "peer-memory gradient exchange was not set up"
        tok = tokens[dp_rank * per_replica : (dp_rank + 1) * per_replica]
        for _ in range(3 if case == "pp_copy" else 2):  # second step exercises the other inbox parity (and the copy transport)
            pipe.zero_grad(set_to_none=False)
            _, loss = pipe(tok[:, :-1].contiguous(), tok[:, 1:].contiguous(), llama_loss_fn, split_size=per_replica // nmb)
        torch.cuda.synchronize()
        gemm.check_status()
        if pipe.is_last():
            assert abs(loss.item() - ref_loss.item()) < 5e-2 * abs(ref_loss.item()), (loss.item(), ref_loss.item())
        worst = 0.0
        for block in pipe.blocks:
            for n, p in block.model.named_parameters():
                e = rel(p.grad, ref_grads[block.id][n])
                worst = max(worst, e)
                assert e < 6e-2, (mode, block.id, n, e)
        results[mode] = worst
        if case == "pp_copy":
            links = [ch.link for ch in pipe.channels.channels.values()]
            assert links and all(l is not None for l in links), "channels did not switch to the copy transport"
            assert any(l.sent > 0 for l in links) and any(l.taken > 0 for l in links)
        if mode == "symm":
            assert all(len(ex.pushed) > 0 for ex in pipe.grad_sync.exchanges.values() if ex is not None), "no gradient left through a GEMM epilogue"
        pipe.clear()
    print(f"rank {rank} case {case} ok: worst relative gradient error {results}", flush=True)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    run(sys.argv[1])
