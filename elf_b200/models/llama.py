"""Llama-style decoder (RMSNorm, RoPE, grouped-query attention, SwiGLU) on this package's
kernels.

The reference's model zoo has no such model (its ``FullTransformer`` is LayerNorm + GELU
without positions, causal mask or GQA; ``benchmarks/models/simple.py:437-468``), but every
benchmark configuration of this project is Llama-shaped.  Layout choices made for the
kernels:

* Q, K and V come from ONE linear layer (``wqkv``) and gate/up from ONE (``w_gate_up``), so
  each decoder layer is four big GEMMs per pass;
* RoPE is applied in place on the fused QKV buffer; attention reads its Q/K/V as strided
  slices of that buffer;
* the residual add after attention is fused into the second RMSNorm;
* all ``nn.Linear`` layers are meant to be wrapped by ``replace_layer_with_layer_dw`` so
  that their weight gradients run as W passes on the tcgen05 GEMM.

Everything falls back to torch ops on CPU / fp32, which is what the numerics tests compare
against.
"""

from __future__ import annotations

from dataclasses import asdict, dataclass
from typing import List, Optional, Sequence

import torch
import torch.nn as nn

from ..ops import attention as _attn
from ..ops import fused as _f

__all__ = [
    "LlamaConfig",
    "LLAMA_CONFIGS",
    "RMSNorm",
    "LlamaEmbedding",
    "LlamaDecoderLayer",
    "LlamaHead",
    "LlamaStage",
    "build_llama_stages",
    "build_llama",
    "llama_loss_fn",
    "init_llama_",
    "layers_per_stage",
    "head_cost_in_layers",
]


@dataclass
class LlamaConfig:
    n_layers: int = 32
    d_model: int = 4096
    n_heads: int = 32
    n_kv_heads: int = 8
    ffn: int = 14336
    vocab: int = 128256
    seq_len: int = 4096
    rope_theta: float = 500000.0
    eps: float = 1e-5
    init_std: float = 0.02

    @property
    def head_dim(self) -> int:
        return self.d_model // self.n_heads

    def n_params(self) -> int:
        d, hd = self.d_model, self.head_dim
        per_layer = d * (self.n_heads + 2 * self.n_kv_heads) * hd + d * d + 3 * d * self.ffn + 2 * d
        return self.n_layers * per_layer + 2 * self.vocab * d + d


LLAMA_CONFIGS = {
    # name: the decoder shapes of the benchmark configurations
    "llama-tiny": LlamaConfig(n_layers=4, d_model=256, n_heads=4, n_kv_heads=2, ffn=512, vocab=1024, seq_len=128, rope_theta=10000.0),
    "llama-1.3b": LlamaConfig(n_layers=24, d_model=2048, n_heads=16, n_kv_heads=16, ffn=5504, vocab=32000, seq_len=2048, rope_theta=10000.0),
    "llama3-8b": LlamaConfig(n_layers=32, d_model=4096, n_heads=32, n_kv_heads=8, ffn=14336, vocab=128256, seq_len=4096, rope_theta=500000.0),
    "llama-13b": LlamaConfig(n_layers=40, d_model=5120, n_heads=40, n_kv_heads=40, ffn=13824, vocab=32000, seq_len=4096, rope_theta=10000.0),
    "llama-70b": LlamaConfig(n_layers=80, d_model=8192, n_heads=64, n_kv_heads=8, ffn=28672, vocab=128256, seq_len=4096, rope_theta=500000.0),
}


class RMSNorm(nn.Module):
    def __init__(self, dim: int, eps: float = 1e-5):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(dim))
        self.eps = eps

    def forward(self, x):
        return _f.rms_norm(x, self.weight, self.eps)


class LlamaEmbedding(nn.Module):
    _elf_leaf = True  # one graph node for the tracers: partitioners cut between layers, not inside

    def __init__(self, cfg: LlamaConfig):
        super().__init__()
        self.weight = nn.Parameter(torch.empty(cfg.vocab, cfg.d_model))

    def forward(self, ids):
        return _f.embedding(self.weight, ids)


class LlamaDecoderLayer(nn.Module):
    _elf_leaf = True

    def __init__(self, cfg: LlamaConfig):
        super().__init__()
        d, hd = cfg.d_model, cfg.head_dim
        self.n_heads, self.n_kv_heads, self.head_dim, self.seq_len = cfg.n_heads, cfg.n_kv_heads, hd, cfg.seq_len
        self.theta = cfg.rope_theta
        self.norm1 = RMSNorm(d, cfg.eps)
        self.wqkv = nn.Linear(d, (cfg.n_heads + 2 * cfg.n_kv_heads) * hd, bias=False)
        self.wo = nn.Linear(cfg.n_heads * hd, d, bias=False)
        self.norm2 = RMSNorm(d, cfg.eps)
        self.w_gate_up = nn.Linear(d, 2 * cfg.ffn, bias=False)
        self.w_down = nn.Linear(cfg.ffn, d, bias=False)
        self._rope = None

    def _tables(self, device, seq_len):
        if self._rope is None or self._rope[0].device != device or self._rope[0].shape[0] < seq_len:
            self._rope = _f.rope_tables(max(seq_len, self.seq_len), self.head_dim, self.theta, device)
        return self._rope

    def forward(self, x):
        b, s, d = x.shape
        hq, hkv, hd = self.n_heads, self.n_kv_heads, self.head_dim
        cos, sin = self._tables(x.device, s)
        # the projection runs on a 2-D view so that its output is a base tensor RoPE may
        # rotate in place
        qkv = self.wqkv(self.norm1(x).view(b * s, d))
        qkv = _f.rope_(qkv, cos, sin, hq + hkv, hd, s).view(b, s, hq + 2 * hkv, hd)
        a = _attn.attention_packed(qkv, hq, hkv, causal=True).reshape(b, s, hq * hd)
        h2, x = _f.add_rms_norm(self.wo(a), x, self.norm2.weight, self.norm2.eps)
        return x + self.w_down(_f.swiglu(self.w_gate_up(h2)))


class LlamaHead(nn.Module):
    _elf_leaf = True

    def __init__(self, cfg: LlamaConfig):
        super().__init__()
        self.norm = RMSNorm(cfg.d_model, cfg.eps)
        self.out = nn.Linear(cfg.d_model, cfg.vocab, bias=False)

    def forward(self, x):
        return self.out(self.norm(x))


class LlamaStage(nn.Sequential):
    """A contiguous run of the model: [embedding] + decoder layers + [head]."""


def init_llama_(module: nn.Module, std: float = 0.02, seed: Optional[int] = None) -> nn.Module:
    """N(0, std) for every matrix, ones for norm gains."""
    gen = None
    for p in module.parameters():
        if p.is_meta:
            continue
        if gen is None and seed is not None:
            gen = torch.Generator(device=p.device).manual_seed(seed)
        if p.dim() >= 2:
            with torch.no_grad():
                p.normal_(0.0, std, generator=gen)
        else:
            with torch.no_grad():
                p.fill_(1.0)
    return module


def head_cost_in_layers(cfg: LlamaConfig) -> float:
    """FLOPs of the LM head (final norm + vocabulary projection) in units of one decoder layer."""
    d, hd = cfg.d_model, cfg.head_dim
    layer = 2 * d * (cfg.n_heads + 2 * cfg.n_kv_heads) * hd + 2 * d * d + 6 * d * cfg.ffn + 2 * cfg.seq_len * d  # last term: causal attention
    return 2 * d * cfg.vocab / layer


def layers_per_stage(n_layers: int, n_stages: int, placement: Optional[Sequence[int]] = None, head_units: float = 0.0) -> List[int]:
    """Decoder-layer count of every stage.

    Without a placement: as even as possible.  With one, the counts balance the work per
    *rank*: the rank hosting the last stage also runs the LM head, which costs ``head_units``
    layers (2.2 for the 8B shape with its 128k vocabulary), so it gets that many fewer layers.
    With a V placement the first and the last stage share a rank, and ignoring this would make
    that rank the bottleneck of the whole pipeline."""
    if placement is None or len(set(placement)) == n_stages == 1:
        base, extra = divmod(n_layers, n_stages)
        return [base + (1 if i < extra else 0) for i in range(n_stages)]
    assert len(placement) == n_stages
    ranks = sorted(set(placement))
    stages_of = {r: [s for s in range(n_stages) if placement[s] == r] for r in ranks}
    head_rank = placement[-1]
    target = (n_layers + head_units) / len(ranks)
    per_rank = {r: 0 for r in ranks}
    per_rank[head_rank] = max(len(stages_of[head_rank]) if n_layers >= n_stages else 0, int(round(target - head_units)))
    others = [r for r in ranks if r != head_rank]
    left = n_layers - per_rank[head_rank]
    if others:
        base, extra = divmod(left, len(others))
        for i, r in enumerate(others):
            per_rank[r] = base + (1 if i < extra else 0)
    else:
        per_rank[head_rank] = n_layers
    counts = [0] * n_stages
    for r in ranks:
        st = stages_of[r]
        base, extra = divmod(per_rank[r], len(st))
        for i, s in enumerate(st):
            counts[s] = base + (1 if i < extra else 0)
    assert sum(counts) == n_layers, (counts, n_layers)
    return counts


def build_llama_stages(cfg: LlamaConfig, n_stages: int, only: Optional[Sequence[int]] = None, device=None, dtype=torch.bfloat16, seed: int = 0, split_backward: bool = True, placement: Optional[Sequence[int]] = None) -> List[Optional[LlamaStage]]:
    """Build the stages listed in ``only`` (all by default) directly on ``device``; the
    others are returned as ``None``, so a rank materialises only what it hosts.  Stage ``i``
    is seeded with ``seed + i``: the weights of a stage do not depend on who builds it.
    With ``placement`` the layer counts are balanced per rank (see ``layers_per_stage``)."""
    from ..zb_utils import replace_layer_with_layer_dw

    counts = layers_per_stage(cfg.n_layers, n_stages, placement, head_cost_in_layers(cfg) if placement is not None else 0.0)
    stages: List[Optional[LlamaStage]] = []
    for i, n in enumerate(counts):
        if only is not None and i not in only:
            stages.append(None)
            continue
        with torch.device(device if device is not None else "cpu"):
            mods: List[nn.Module] = []
            if i == 0:
                mods.append(LlamaEmbedding(cfg))
            mods += [LlamaDecoderLayer(cfg) for _ in range(n)]
            if i == n_stages - 1:
                mods.append(LlamaHead(cfg))
            stage = LlamaStage(*mods).to(dtype)
        init_llama_(stage, cfg.init_std, seed + i)
        if split_backward:
            replace_layer_with_layer_dw(stage)
        stages.append(stage)
    return stages


def build_llama(cfg: LlamaConfig, device=None, dtype=torch.bfloat16, seed: int = 0, split_backward: bool = False) -> nn.Sequential:
    """The whole model as one flat ``nn.Sequential`` (for tracing / single-device use)."""
    (stage,) = build_llama_stages(cfg, 1, device=device, dtype=dtype, seed=seed, split_backward=split_backward)
    return stage


def llama_loss_fn(logits, target, reduction: str = "mean"):
    """Next-token cross entropy; consumes the logits buffer on the CUDA path."""
    return _f.cross_entropy(logits, target, reduction=reduction)
