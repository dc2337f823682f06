"""A Llama-style decoder under ZB-V, with both the stage cut and the schedule made from
measurements: block times timed on the device decide where the stages are cut (inside layers
where that balances better), and the schedule is laid out again for the per-stage times of a
warm-up step.

    torchrun --nproc-per-node 4 examples/llama_zbv_profile_guided.py            # 4 GPUs (or CPU ranks)
    torchrun --nproc-per-node 2 examples/llama_zbv_profile_guided.py --name llama-tiny

On CPU ranks the block times come from the built-in constants instead of a measurement.
"""

import argparse
import functools
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from elf_b200 import Pipeline, Placement  # noqa: E402
from elf_b200.models.llama import LLAMA_CONFIGS, build_llama_stages, choose_llama_cut, llama_loss_fn, llama_stage_signatures  # noqa: E402
from elf_b200.models.llama_costs import measure_cost_model  # noqa: E402
from elf_b200.optim import FusedAdamW  # noqa: E402
from elf_b200.scheduling.schedulers import generate_zbv_schedule  # noqa: E402

ap = argparse.ArgumentParser()
ap.add_argument("--name", default="llama-tiny", choices=sorted(LLAMA_CONFIGS))
ap.add_argument("--nmb", type=int, default=8, help="micro-batches per step")
ap.add_argument("--steps", type=int, default=4)
args = ap.parse_args()

use_cuda = torch.cuda.is_available()
if use_cuda:
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", 0)))
dist.init_process_group("nccl" if use_cuda else "gloo")
rank, world = dist.get_rank(), dist.get_world_size()
device = torch.device("cuda", torch.cuda.current_device()) if use_cuda else torch.device("cpu")
dtype = torch.bfloat16 if use_cuda else torch.float32

cfg = LLAMA_CONFIGS[args.name]
placement = list(Placement.default("zbv", world))  # [0..p-1, p-1..0]: two stages per rank
n_stages = len(placement)

# 1. what the parts of a layer, the embedding and the head cost on this device (rank 0 measures, all ranks get the result)
cost_model = measure_cost_model(cfg, device, mb_size=1)
cost_model.micro_batches = args.nmb  # lets the cut allow for the pipeline's fill
# 2. cut between attention and MLP halves, or also inside the MLP when the simulated step gains from it
cut = dict(placement=placement, split_layers=choose_llama_cut(cfg, n_stages, placement, cost_model), cost_model=cost_model)
mine = Placement(placement).get_ids(rank)
stages = build_llama_stages(cfg, n_stages, only=mine, device=device, dtype=dtype, seed=0, **cut)
pipe = Pipeline([stages[i] for i in mine], None, partitioner=False, scheduler="zbv", placement=placement, outputs="none",
                signatures=llama_stage_signatures(cfg, n_stages, **cut))
params = list(pipe.parameters())
opt = FusedAdamW(params, lr=3e-4) if params else None

gen = torch.Generator().manual_seed(0)
for step in range(args.steps):
    tokens = torch.randint(0, cfg.vocab, (args.nmb, cfg.seq_len + 1), generator=gen).to(device)
    if step == 1:
        os.environ["ELF_TIMINGS"] = "1"  # time every operation of this step
    pipe.zero_grad()
    _, loss = pipe(tokens[:, :-1].contiguous(), tokens[:, 1:].contiguous(), llama_loss_fn, split_size=1)
    if opt is not None:
        opt.step()
    if step == 1:
        os.environ.pop("ELF_TIMINGS")
        # 3. lay ZB-V out again for the measured (forward, input-gradient, weight-gradient) time of every stage
        measured = pipe.measured_stage_costs()
        pipe.set_scheduler(functools.partial(generate_zbv_schedule, cap="auto", stage_costs=measured, robust=0.02))
    if pipe.is_last():
        print(f"step {step}: loss {loss.item():.4f}")
pipe.clear()
dist.destroy_process_group()
