"""GPT-style decoder (LayerNorm, GELU MLP, learned positions, causal MHA) built from stock
torch ops.  Used for CPU/gloo plumbing tests and as a small example model; the Llama family
in ``elf_b200.models.llama`` is the one that runs on the sm_100a kernels."""

from __future__ import annotations

from dataclasses import dataclass
from typing import List

import torch
import torch.nn as nn
import torch.nn.functional as F

__all__ = ["GPTConfig", "GPTEmbedding", "GPTBlock", "GPTHead", "GPT", "gpt_stages"]


@dataclass
class GPTConfig:
    n_layers: int = 4
    d_model: int = 256
    n_heads: int = 4
    ffn: int = 1024
    vocab: int = 1024
    seq_len: int = 128
    init_std: float = 0.02


class GPTEmbedding(nn.Module):
    def __init__(self, cfg: GPTConfig):
        super().__init__()
        self.tok = nn.Embedding(cfg.vocab, cfg.d_model)
        self.pos = nn.Embedding(cfg.seq_len, cfg.d_model)

    def forward(self, ids):
        pos = torch.arange(ids.size(1), device=ids.device)
        return self.tok(ids) + self.pos(pos)[None]


class GPTBlock(nn.Module):
    def __init__(self, cfg: GPTConfig):
        super().__init__()
        self.n_heads = cfg.n_heads
        self.ln1 = nn.LayerNorm(cfg.d_model)
        self.qkv = nn.Linear(cfg.d_model, 3 * cfg.d_model)
        self.proj = nn.Linear(cfg.d_model, cfg.d_model)
        self.ln2 = nn.LayerNorm(cfg.d_model)
        self.fc1 = nn.Linear(cfg.d_model, cfg.ffn)
        self.fc2 = nn.Linear(cfg.ffn, cfg.d_model)

    def forward(self, x):
        b, s, d = x.shape
        q, k, v = self.qkv(self.ln1(x)).view(b, s, 3, self.n_heads, d // self.n_heads).permute(2, 0, 3, 1, 4)
        a = F.scaled_dot_product_attention(q, k, v, is_causal=True)
        x = x + self.proj(a.transpose(1, 2).reshape(b, s, d))
        return x + self.fc2(F.gelu(self.fc1(self.ln2(x))))


class GPTHead(nn.Module):
    def __init__(self, cfg: GPTConfig):
        super().__init__()
        self.ln = nn.LayerNorm(cfg.d_model)
        self.out = nn.Linear(cfg.d_model, cfg.vocab, bias=False)

    def forward(self, x):
        return self.out(self.ln(x))


def _init(module: nn.Module, std: float) -> None:
    for m in module.modules():
        if isinstance(m, (nn.Linear, nn.Embedding)):
            nn.init.normal_(m.weight, 0.0, std)
            if getattr(m, "bias", None) is not None:
                nn.init.zeros_(m.bias)


class GPT(nn.Sequential):
    """Embedding, ``n_layers`` blocks, head — as a flat ``nn.Sequential`` so it can be cut
    anywhere."""

    def __init__(self, cfg: GPTConfig):
        super().__init__(GPTEmbedding(cfg), *[GPTBlock(cfg) for _ in range(cfg.n_layers)], GPTHead(cfg))
        self.cfg = cfg
        _init(self, cfg.init_std)

    @staticmethod
    def loss_fn(logits, target, reduction="mean"):
        return F.cross_entropy(logits.float().view(-1, logits.size(-1)), target.reshape(-1), reduction=reduction)


def gpt_stages(model: nn.Sequential, n_stages: int) -> List[nn.Sequential]:
    """Split a flat sequential model into ``n_stages`` contiguous chunks of balanced length."""
    layers = list(model.children())
    base, extra = divmod(len(layers), n_stages)
    out, start = [], 0
    for i in range(n_stages):
        n = base + (1 if i < extra else 0)
        out.append(nn.Sequential(*layers[start : start + n]))
        start += n
    return out
