"""Reference arm of ``bench.py``: the UNMODIFIED reference package (installed offline into
``baseline/_ref``) training the same Llama-shaped decoder on the same synthetic data,
through its own public API and stock code path.

Nothing of ``elf_b200`` is imported here.  The model is written with stock torch ops only
(``nn.Linear``, ``F.rms_norm``, RoPE from cos/sin tables, ``F.scaled_dot_product_attention``
with ``enable_gqa``, ``F.silu``, fp32 ``F.cross_entropy``), because the reference's own model
zoo cannot express RMSNorm/RoPE/GQA/SwiGLU.  It is handed to ``elf.Pipeline`` pre-partitioned
(``partitioner=False`` + ``sequential_signatures``), its linear layers wrapped by the
reference's ``replace_layer_with_layer_dw``; the optimizer is ``torch.optim.AdamW(fused=True)``
on the bf16 parameters, stepped inside the timed region.

Known limits of the reference that shape this arm:
* its ZB-V generator only supports ``nmb == 2 * pp``; with 16 micro-batches that is pp = 8.
  For other GPU counts the arm runs ZB-H1, the other schedule the configuration names;
* every micro-batch's logits are copied to the host by its engine (stock behaviour).
"""

from __future__ import annotations

import json
import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
REF_DIR = os.path.join(HERE, "_ref")

_CONFIGS = {
    "llama-tiny": dict(n_layers=4, d_model=256, n_heads=4, n_kv_heads=2, ffn=512, vocab=1024, seq_len=128, rope_theta=10000.0),
    "llama-1.3b": dict(n_layers=24, d_model=2048, n_heads=16, n_kv_heads=16, ffn=5504, vocab=32000, seq_len=2048, rope_theta=10000.0),
    "llama3-8b": dict(n_layers=32, d_model=4096, n_heads=32, n_kv_heads=8, ffn=14336, vocab=128256, seq_len=4096, rope_theta=500000.0),
}


def _layers_per_stage(c, placement):
    """Layer counts balancing the work per RANK: the rank with the last stage also runs the LM
    head, which costs `head` decoder layers.  (Same rule as the other arm of the benchmark,
    restated here because this file imports nothing from it.)"""
    n_layers, n_stages = c["n_layers"], len(placement)
    d, hd = c["d_model"], c["d_model"] // c["n_heads"]
    layer = 2 * d * (c["n_heads"] + 2 * c["n_kv_heads"]) * hd + 2 * d * d + 6 * d * c["ffn"] + 2 * c["seq_len"] * d
    head = 2 * d * c["vocab"] / layer
    ranks = sorted(set(placement))
    stages_of = {r: [s for s in range(n_stages) if placement[s] == r] for r in ranks}
    head_rank = placement[-1]
    per_rank = {r: 0 for r in ranks}
    if len(ranks) == 1:
        per_rank[head_rank] = n_layers
    else:
        target = (n_layers + head) / len(ranks)
        per_rank[head_rank] = max(len(stages_of[head_rank]) if n_layers >= n_stages else 0, int(round(target - head)))
        others = [r for r in ranks if r != head_rank]
        base, extra = divmod(n_layers - per_rank[head_rank], len(others))
        for i, r in enumerate(others):
            per_rank[r] = base + (1 if i < extra else 0)
    counts = [0] * n_stages
    for r in ranks:
        st = stages_of[r]
        base, extra = divmod(per_rank[r], len(st))
        for i, s in enumerate(st):
            counts[s] = base + (1 if i < extra else 0)
    assert sum(counts) == n_layers
    return counts


def _unavailable(why: str) -> None:
    print(json.dumps({"impl": "reference", "unavailable": why}), flush=True)


def _build_modules(torch, nn, F):
    class RefLayer(nn.Module):
        def __init__(self, c):
            super().__init__()
            d, hd = c["d_model"], c["d_model"] // c["n_heads"]
            self.hq, self.hkv, self.hd, self.theta, self.eps = c["n_heads"], c["n_kv_heads"], hd, c["rope_theta"], 1e-5
            self.g1 = nn.Parameter(torch.ones(d))
            self.wqkv = nn.Linear(d, (self.hq + 2 * self.hkv) * hd, bias=False)
            self.wo = nn.Linear(self.hq * hd, d, bias=False)
            self.g2 = nn.Parameter(torch.ones(d))
            self.w_gate_up = nn.Linear(d, 2 * c["ffn"], bias=False)
            self.w_down = nn.Linear(c["ffn"], d, bias=False)
            self._tables = None

        def tables(self, s, device, dtype):
            if self._tables is None or self._tables[0].shape[0] < s or self._tables[0].device != device:
                inv = 1.0 / (self.theta ** (torch.arange(0, self.hd, 2, dtype=torch.float64) / self.hd))
                ang = torch.outer(torch.arange(s, dtype=torch.float64), inv)
                self._tables = (ang.cos().to(device=device, dtype=dtype), ang.sin().to(device=device, dtype=dtype))
            return self._tables

        def rope(self, t, cos, sin):
            half = self.hd // 2
            a, b = t[..., :half], t[..., half:]
            c, s = cos[None, :, None, :], sin[None, :, None, :]
            return torch.cat([a * c - b * s, b * c + a * s], dim=-1)

        def forward(self, x):
            b, s, d = x.shape
            h = F.rms_norm(x, (d,), self.g1, self.eps)
            qkv = self.wqkv(h).view(b, s, self.hq + 2 * self.hkv, self.hd)
            q, k, v = qkv[:, :, : self.hq], qkv[:, :, self.hq : self.hq + self.hkv], qkv[:, :, self.hq + self.hkv :]
            cos, sin = self.tables(s, x.device, x.dtype)
            q, k = self.rope(q, cos[:s], sin[:s]), self.rope(k, cos[:s], sin[:s])
            a = F.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), is_causal=True, enable_gqa=self.hq != self.hkv)
            x = x + self.wo(a.transpose(1, 2).reshape(b, s, self.hq * self.hd))
            h = F.rms_norm(x, (d,), self.g2, self.eps)
            g, u = self.w_gate_up(h).chunk(2, dim=-1)
            return x + self.w_down(F.silu(g) * u)

    class RefEmbed(nn.Module):
        def __init__(self, c):
            super().__init__()
            self.emb = nn.Embedding(c["vocab"], c["d_model"])

        def forward(self, ids):
            return self.emb(ids)

    class RefHead(nn.Module):
        def __init__(self, c):
            super().__init__()
            self.g = nn.Parameter(torch.ones(c["d_model"]))
            self.out = nn.Linear(c["d_model"], c["vocab"], bias=False)

        def forward(self, x):
            return self.out(F.rms_norm(x, (x.shape[-1],), self.g, 1e-5))

    return RefLayer, RefEmbed, RefHead


def run_reference(args) -> None:
    if not os.path.isdir(os.path.join(REF_DIR, "elf")):
        return _unavailable("baseline/_ref/elf is missing: the offline install of the reference has not been run")
    sys.path.insert(0, REF_DIR)
    try:
        import torch
        import torch.distributed as dist
        import torch.nn as nn
        import torch.nn.functional as F

        if not torch.cuda.is_available():
            return _unavailable("the reference calls torch.cuda unconditionally and there is no GPU")
        import elf  # the reference package
        from elf import Pipeline, sequential_signatures, replace_layer_with_layer_dw
        from elf.utils import Placement
    except Exception as exc:  # import problems are reported, not raised
        return _unavailable(f"cannot import the reference: {type(exc).__name__}: {exc}")
    assert os.path.realpath(elf.__file__).startswith(os.path.realpath(REF_DIR)), elf.__file__

    rank = int(os.environ.get("RANK", 0))
    world = int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", rank))
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29533")
    os.environ.setdefault("RANK", "0")
    os.environ.setdefault("WORLD_SIZE", "1")
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=device)
    if world != args.gpus:
        return _unavailable(f"--gpus {args.gpus} but WORLD_SIZE={world}")

    c = dict(_CONFIGS[args.model])
    if args.seq_len:
        c["seq_len"] = args.seq_len
    if args.layers:
        c["n_layers"] = args.layers
    pp = world // args.dp
    scheduler = args.scheduler
    note = None
    if scheduler == "zbv" and args.nmb != 2 * pp:
        scheduler = "zbh1"
        note = f"reference ZB-V supports only nmb == 2*pp (nmb={args.nmb}, pp={pp}); ran ZB-H1 instead"
    if args.dp > 1 and scheduler in ("1f1b", "megatron", "zbv", "hanayo"):
        return _unavailable(f"the reference's {scheduler} schedule is empty or raises IndexError on replicas other than the first (dp={args.dp})")
    placement = Placement.default(scheduler, pp)
    n_stages = len(placement)
    counts = _layers_per_stage(c, list(placement))
    RefLayer, RefEmbed, RefHead = _build_modules(torch, nn, F)
    mine = [i for i in range(n_stages) if placement[i] == rank % pp]
    parts = []
    for i in mine:
        with torch.device(device):
            mods = ([RefEmbed(c)] if i == 0 else []) + [RefLayer(c) for _ in range(counts[i])] + ([RefHead(c)] if i == n_stages - 1 else [])
            stage = nn.Sequential(*mods).to(torch.bfloat16)
        gen = torch.Generator(device=device).manual_seed(1234 + i)
        with torch.no_grad():
            for p in stage.parameters():
                if p.dim() >= 2:
                    p.normal_(0.0, 0.02, generator=gen)
        replace_layer_with_layer_dw(stage)
        parts.append(stage)

    def loss_fn(logits, target, reduction="mean"):
        return F.cross_entropy(logits.float().view(-1, logits.size(-1)), target.reshape(-1), reduction=reduction)

    try:
        pipe = Pipeline(parts, None, partitioner=False, scheduler=scheduler, placement=list(placement), dp=args.dp, signatures=sequential_signatures(placement))
        params = list(pipe.parameters())
        opt = torch.optim.AdamW(params, lr=1e-4, betas=(0.9, 0.95), eps=1e-5, weight_decay=0.1, fused=True) if params else None

        batch = args.nmb * args.mb_size
        n_batches = args.warmup + 2 * args.steps
        gen = torch.Generator().manual_seed(1000 + rank // pp)
        host = [torch.randint(0, c["vocab"], (batch, c["seq_len"] + 1), generator=gen).pin_memory() for _ in range(n_batches)]

        def to_device(tok):
            tok = tok.to(device, non_blocking=True)
            return tok[:, :-1].contiguous(), tok[:, 1:].contiguous()

        def step(ids, tgt):
            if opt is not None:
                opt.zero_grad()
            else:
                pipe.zero_grad()
            _, loss = pipe(ids, tgt, loss_fn, split_size=args.mb_size)
            if opt is not None:
                opt.step()
            return loss

        def fence():
            torch.cuda.synchronize()
            dist.barrier()
            torch.cuda.synchronize()

        def max_ranks(v):
            t = torch.tensor([v], dtype=torch.float64, device=device)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            return float(t.item())

        from benchmarks.benchmark_utils import ClockSampler  # nvidia-smi reader only; no kernels, no engine

        it = iter(host)
        loss = None
        for _ in range(args.warmup):
            loss = step(*to_device(next(it)))
        resident = [to_device(next(it)) for _ in range(args.steps)]
        fence()
        torch.cuda.reset_peak_memory_stats()
        with ClockSampler(local) as clocks:
            start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
            for ids, tgt in resident:
                loss = step(ids, tgt)
            end.record()
            fence()
        dev_ms = max_ranks(start.elapsed_time(end))
        peak_gb = max_ranks(torch.cuda.max_memory_allocated() / 2**30)
        last_loss = float(loss.item()) if loss is not None else None
        del resident
        e2e = None
        if not args.no_e2e:
            fence()
            start.record()
            for _ in range(args.steps):
                loss = step(*to_device(next(it)))
                if loss is not None:
                    last_loss = float(loss.item())
            end.record()
            fence()
            e2e_ms = max_ranks(start.elapsed_time(end))
            tokens = args.dp * batch * c["seq_len"] * args.steps
            # bytes of the whole job per step: every rank copies its batch of token ids to its GPU
            # (only the ranks hosting the first and the last stage read them), the rank that owns
            # the loss reads it back; summed over ranks so that the line does not depend on which
            # rank prints it
            io = torch.tensor([int(host[0].numel() * host[0].element_size()), 4 if placement[-1] == rank % pp else 0], dtype=torch.float64, device=device)
            dist.all_reduce(io, op=dist.ReduceOp.SUM)
            e2e = {
                "value": tokens / (e2e_ms / 1e3),
                "unit": "tokens/s",
                "ms_per_step": e2e_ms / args.steps,
                "h2d_bytes_per_step": int(io[0].item()),
                "d2h_bytes_per_step": int(io[1].item()),
            }
    except torch.cuda.OutOfMemoryError as exc:
        return _unavailable(f"reference ran out of GPU memory on this configuration: {str(exc)[:120]}")
    except (AssertionError, IndexError, RuntimeError) as exc:
        return _unavailable(f"reference failed on this configuration: {type(exc).__name__}: {str(exc)[:160]}")

    tokens = args.dp * batch * c["seq_len"] * args.steps
    line = {
        "metric": "training throughput, tokens/sec (device-timed, max over ranks)",
        "impl": "reference",
        "value": tokens / (dev_ms / 1e3),
        "unit": "tokens/s",
        "n_gpus": world,
        "steps": args.steps,
        "warmup": args.warmup,
        "ms_per_step": dev_ms / args.steps,
        "higher_is_better": True,
        "scaling": "strong",
        "vs_baseline": None,
        "dtype": "bf16",
        "data": "synthetic uniform token ids, N(0,0.02) random-init weights",
        "config": {
            "model": f"{args.model} ({c['n_layers']} layers, d={c['d_model']}, {c['n_heads']}q/{c['n_kv_heads']}kv heads, ffn={c['ffn']}, vocab={c['vocab']})",
            "global_batch": args.dp * batch,
            "micro_batches": args.nmb,
            "micro_batch_size": args.mb_size,
            "seq_len": c["seq_len"],
            "parallelism": f"pp{pp}" + (f"xdp{args.dp}" if args.dp > 1 else ""),
            "scheduler": scheduler,
            "placement": list(placement),
            "layers_per_stage": counts,
            "optimizer": "torch.optim.AdamW(fused=True) on bf16 parameters, step inside the timed region",
            "note": note,
        },
        "clocks": clocks.summary(),
        "e2e": e2e,
        "gpu_launches": 0,
        "peak_gb_per_gpu": peak_gb,
        "loss": last_loss,
    }
    if rank == 0:
        print(json.dumps(line), flush=True)
    dist.barrier()
    dist.destroy_process_group()
