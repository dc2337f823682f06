"""Manual partitioning: every rank builds its own stage, Zero-Bubble (ZB-H2) schedule with
split-backward linear layers.

    torchrun --nproc-per-node 4 examples/basic_no_partition.py
"""

import os
import sys

import torch
import torch.distributed as dist
import torch.nn as nn

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from elf_b200 import Pipeline, Placement, replace_layer_with_layer_dw, sequential_signatures  # noqa: E402

use_cuda = torch.cuda.is_available()
if use_cuda:
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", 0)))
dist.init_process_group("nccl" if use_cuda else "gloo")
rank, world = dist.get_rank(), dist.get_world_size()
device = "cuda" if use_cuda else "cpu"

torch.manual_seed(rank)
stage = nn.Sequential(nn.Linear(256, 1024), nn.GELU(), nn.Linear(1024, 256)).to(device)
replace_layer_with_layer_dw(stage)  # weight gradients become separate W passes
placement = Placement.linear(world)
pipe = Pipeline(stage, None, partitioner=False, scheduler="zbh2", placement=placement, signatures=sequential_signatures(placement))
opt = torch.optim.AdamW(pipe.parameters(), lr=1e-3)

for step in range(5):
    x = torch.randn(16, 256, device=device)
    opt.zero_grad()
    _, loss = pipe(x, x, nn.functional.mse_loss, split_size=2)
    opt.step()
    if pipe.is_last():
        print(f"step {step}: loss {loss.item():.4f}")
pipe.clear()
dist.destroy_process_group()
