"""Small model zoo used by examples, tests and the benchmark CLI (counterpart of the
reference's ``benchmarks/models/simple.py``): feed-forward, residual CNN, attention blocks,
a pre-LN GELU transformer (``FullTransformer`` / ``ChainTransformer``).  Every model exposes
``get_sample``, ``get_target`` and ``loss_fn``.  All of it is stock torch; the Llama family
(``elf_b200.models.llama``) is what runs on the sm_100a kernels."""

from __future__ import annotations

from typing import Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

__all__ = [
    "SimpleFFN",
    "SimpleResNet",
    "SimpleCNN",
    "Attention",
    "MultiHeadAttention",
    "TransformerBlock",
    "FullTransformer",
    "ChainTransformer",
]


class _SampleMixin:
    def get_target(self, batch_size: int, dtype=torch.float32, device="cpu"):
        return self.get_sample(batch_size, dtype, device)

    @staticmethod
    def loss_fn(out, target, reduction: str = "mean"):
        return F.mse_loss(out.float(), target.float(), reduction=reduction)


class SimpleFFN(nn.Module, _SampleMixin):
    def __init__(self, input_dim: int = 64, hidden_dim: int = 256, n_blocks: int = 8):
        super().__init__()
        self.input_dim = input_dim
        layers = []
        for _ in range(n_blocks):
            layers += [nn.Linear(input_dim, hidden_dim), nn.GELU(), nn.Linear(hidden_dim, input_dim)]
        self.layers = nn.Sequential(*layers)

    def forward(self, x):
        return self.layers(x)

    def get_sample(self, batch_size, dtype=torch.float32, device="cpu"):
        return torch.randn(batch_size, self.input_dim, dtype=dtype, device=device)


class _ResBlock(nn.Module):
    def __init__(self, c):
        super().__init__()
        self.c1, self.c2 = nn.Conv2d(c, c, 3, padding=1), nn.Conv2d(c, c, 3, padding=1)
        self.b1, self.b2 = nn.BatchNorm2d(c), nn.BatchNorm2d(c)

    def forward(self, x):
        return F.relu(x + self.b2(self.c2(F.relu(self.b1(self.c1(x))))))


class SimpleResNet(nn.Module, _SampleMixin):
    def __init__(self, channels: int = 16, n_blocks: int = 4, n_classes: int = 10, image: int = 32):
        super().__init__()
        self.image = image
        self.stem = nn.Conv2d(3, channels, 3, padding=1)
        self.blocks = nn.Sequential(*[_ResBlock(channels) for _ in range(n_blocks)])
        self.head = nn.Linear(channels, n_classes)

    def forward(self, x):
        return self.head(self.blocks(self.stem(x)).mean(dim=(2, 3)))

    def get_sample(self, batch_size, dtype=torch.float32, device="cpu"):
        return torch.randn(batch_size, 3, self.image, self.image, dtype=dtype, device=device)

    def get_target(self, batch_size, dtype=torch.float32, device="cpu"):
        return torch.randint(0, self.head.out_features, (batch_size,), device=device)

    @staticmethod
    def loss_fn(out, target, reduction="mean"):
        return F.cross_entropy(out.float(), target, reduction=reduction)


class SimpleCNN(SimpleResNet):
    """Plain stack of 3x3 convolutions (no skip connections)."""

    def __init__(self, channels: int = 16, n_blocks: int = 4, n_classes: int = 10, image: int = 32):
        super().__init__(channels, 0, n_classes, image)
        self.blocks = nn.Sequential(*[m for _ in range(n_blocks) for m in (nn.Conv2d(channels, channels, 3, padding=1), nn.ReLU())])


class Attention(nn.Module):
    """Multi-head self-attention through ``F.scaled_dot_product_attention``."""

    def __init__(self, hidden_dim: int, num_heads: int, dropout: float = 0.0, causal: bool = False):
        super().__init__()
        self.h, self.p, self.causal = num_heads, dropout, causal
        self.q, self.k, self.v = (nn.Linear(hidden_dim, hidden_dim) for _ in range(3))
        self.proj = nn.Linear(hidden_dim, hidden_dim)

    def forward(self, x):
        b, s, d = x.shape
        shape = lambda t: t.view(b, s, self.h, d // self.h).transpose(1, 2)
        a = F.scaled_dot_product_attention(shape(self.q(x)), shape(self.k(x)), shape(self.v(x)), dropout_p=self.p if self.training else 0.0, is_causal=self.causal)
        return self.proj(a.transpose(1, 2).reshape(b, s, d))


MultiHeadAttention = Attention


class TransformerBlock(nn.Module):
    def __init__(self, hidden_dim: int, num_heads: int, ffn_dim: int, dropout: float = 0.0, causal: bool = False):
        super().__init__()
        self.ln1, self.ln2 = nn.LayerNorm(hidden_dim), nn.LayerNorm(hidden_dim)
        self.attn = Attention(hidden_dim, num_heads, dropout, causal)
        self.fc1, self.fc2 = nn.Linear(hidden_dim, ffn_dim), nn.Linear(ffn_dim, hidden_dim)
        self.drop = nn.Dropout(dropout)

    def forward(self, x):
        x = x + self.drop(self.attn(self.ln1(x)))
        return x + self.drop(self.fc2(F.gelu(self.fc1(self.ln2(x)))))


class TokenEmbedding(nn.Module):
    """Token embedding plus learned positions: one module, so that a hand-made first stage
    (``nn.Sequential(model.embed, *blocks)``) computes what the whole model computes."""

    def __init__(self, vocab: int, hidden_dim: int, seq_len: int):
        super().__init__()
        self.tok = nn.Embedding(vocab, hidden_dim)
        self.pos = nn.Embedding(seq_len, hidden_dim)

    def forward(self, ids):
        return self.tok(ids) + self.pos(torch.arange(ids.size(1), device=ids.device))[None]


class FullTransformer(nn.Module):
    """Embedding + pre-LN GELU blocks + LM head; cross-entropy in fp32."""

    def __init__(self, input_dim: int = 1024, hidden_dim: int = 256, n_blocks: int = 4, seq_len: int = 128, num_heads: int = 4, ffn_dim: Optional[int] = None, dropout: float = 0.0, causal: bool = True, **_unused):
        super().__init__()
        self.vocab, self.seq_len = input_dim, seq_len
        self.embed = TokenEmbedding(input_dim, hidden_dim, seq_len)
        self.blocks = nn.Sequential(*[TransformerBlock(hidden_dim, num_heads, ffn_dim or 4 * hidden_dim, dropout, causal) for _ in range(n_blocks)])
        self.ln = nn.LayerNorm(hidden_dim)
        self.head = nn.Linear(hidden_dim, input_dim, bias=False)

    def forward(self, ids):
        return self.head(self.ln(self.blocks(self.embed(ids))))

    def get_sample(self, batch_size, dtype=None, device="cpu"):
        return torch.randint(0, self.vocab, (batch_size, self.seq_len), device=device)

    get_target = get_sample

    @staticmethod
    def loss_fn(out, target, reduction="mean"):
        return F.cross_entropy(out.float().reshape(-1, out.size(-1)), target.reshape(-1), reduction=reduction)


class ChainTransformer(nn.Module, _SampleMixin):
    """Transformer blocks on float inputs, no embedding or head."""

    def __init__(self, hidden_dim: int = 256, n_blocks: int = 4, seq_len: int = 128, num_heads: int = 4, ffn_dim: Optional[int] = None, dropout: float = 0.0, **_unused):
        super().__init__()
        self.hidden_dim, self.seq_len = hidden_dim, seq_len
        self.blocks = nn.Sequential(*[TransformerBlock(hidden_dim, num_heads, ffn_dim or 4 * hidden_dim, dropout) for _ in range(n_blocks)])

    def forward(self, x):
        return self.blocks(x)

    def get_sample(self, batch_size, dtype=torch.float32, device="cpu"):
        return torch.randn(batch_size, self.seq_len, self.hidden_dim, dtype=dtype, device=device)
