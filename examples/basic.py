"""Automatic partitioning: trace a model, cut it into one stage per rank, train with 1F1B.

    torchrun --nproc-per-node 2 examples/basic.py          # GPUs (NCCL) or CPUs (gloo)
"""

import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from elf_b200 import Pipeline  # noqa: E402
from elf_b200.models.simple import SimpleResNet  # noqa: E402

use_cuda = torch.cuda.is_available()
if use_cuda:
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", 0)))
dist.init_process_group("nccl" if use_cuda else "gloo")
device = "cuda" if use_cuda else "cpu"

torch.manual_seed(0)
model = SimpleResNet(channels=16, n_blocks=6)
sample = model.get_sample(2, device=device)  # one micro-batch
pipe = Pipeline(model.to(device) if dist.get_rank() == 0 else model, sample, scheduler="1f1b")
opt = torch.optim.SGD(pipe.parameters(), lr=0.05)

for step in range(5):
    x, y = model.get_sample(8, device=device), model.get_target(8, device=device)
    opt.zero_grad()
    _, loss = pipe(x, y, SimpleResNet.loss_fn, split_size=2)
    opt.step()
    if pipe.is_last():
        print(f"step {step}: loss {loss.item():.4f}")
pipe.clear()
dist.destroy_process_group()
