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
    "FeedForward",
    "scaled_dot_product",
    "SDP_BACKENDS",
    "Attention",
    "FastAttention",
    "MultiHeadAttention",
    "SimpleAttention",
    "SimpleFastAttention",
    "SimpleTransformer",
    "TransformerBlock",
    "TokenEmbedding",
    "FullTransformer",
    "ChainTransformer",
    "make_simple_fno",
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


class FeedForward(nn.Module):
    def __init__(self, hidden_dim: int, ffn_dim: int, activation=nn.GELU):
        super().__init__()
        self.fc1, self.act, self.fc2 = nn.Linear(hidden_dim, ffn_dim), activation(), nn.Linear(ffn_dim, hidden_dim)

    def forward(self, x):
        return self.fc2(self.act(self.fc1(x)))


# Names accepted for ``sdp_backend`` (the reference's ``--sdp-backend`` choices,
# ``benchmarks/models/utils.py:186-192``, plus this package's own kernels):
#   None / "none"    whatever ``F.scaled_dot_product_attention`` picks
#   "MATH", "FLASH_ATTENTION", "EFFICIENT_ATTENTION", "CUDNN_ATTENTION"   one torch SDPA backend
#   "fatt3"          the flash-attn package, when it is installed
#   "native"         the tcgen05 kernels of ``elf_b200.ops.attention_native`` (causal, bf16/fp16, head_dim 128)
SDP_BACKENDS = (None, "MATH", "FLASH_ATTENTION", "EFFICIENT_ATTENTION", "CUDNN_ATTENTION", "fatt3", "native")


def scaled_dot_product(q, k, v, sdp_backend: Optional[str] = None, dropout_p: float = 0.0, causal: bool = False):
    """Attention over ``[batch, heads, seq, head_dim]`` tensors through the chosen back end."""
    if sdp_backend in (None, "none"):
        return F.scaled_dot_product_attention(q, k, v, dropout_p=dropout_p, is_causal=causal, enable_gqa=q.size(1) != k.size(1))
    if sdp_backend == "fatt3":
        try:
            from flash_attn import flash_attn_func
        except ImportError as exc:
            raise RuntimeError("sdp_backend='fatt3' needs the flash-attn package") from exc
        return flash_attn_func(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), dropout_p=dropout_p, causal=causal).transpose(1, 2)
    if sdp_backend == "native":
        from ..ops.attention_native import native_applicable_packed, native_attention_packed

        if not causal or dropout_p:
            raise RuntimeError("sdp_backend='native' implements causal attention without dropout")
        b, h, s_, d = q.shape
        qkv = torch.cat([q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2)], dim=2).contiguous()  # the kernels read one packed [b, s, hq + 2 hkv, d] buffer
        if not native_applicable_packed(qkv, h, k.size(1), causal):
            raise RuntimeError("sdp_backend='native' needs CUDA bf16/fp16 tensors with head_dim 128 and a sequence length that is a multiple of 128")
        return native_attention_packed(qkv, h, k.size(1)).transpose(1, 2)
    from torch.nn.attention import SDPBackend, sdpa_kernel

    if not hasattr(SDPBackend, sdp_backend):
        raise ValueError(f"unknown sdp_backend {sdp_backend!r}; choose from {SDP_BACKENDS}")
    with sdpa_kernel(backends=[getattr(SDPBackend, sdp_backend)]):
        return F.scaled_dot_product_attention(q, k, v, dropout_p=dropout_p, is_causal=causal, enable_gqa=q.size(1) != k.size(1))


class Attention(nn.Module):
    """Attention core written out as matmul / softmax / matmul (no fused kernel): the slow
    baseline the fused back ends are compared with.  Takes and returns ``[b, h, s, d]``."""

    def __init__(self, dropout: float = 0.0, causal: bool = False):
        super().__init__()
        self.dropout, self.causal = dropout, causal

    def forward(self, q, k, v):
        scores = (q @ k.transpose(-2, -1)) / (q.size(-1) ** 0.5)
        if self.causal:
            s_ = scores.size(-1)
            scores = scores.masked_fill(torch.ones(s_, s_, dtype=torch.bool, device=q.device).triu(1), float("-inf"))
        w = F.dropout(scores.softmax(-1), self.dropout, self.training)
        return w @ v


class FastAttention(nn.Module):
    """Attention core on a fused back end (see ``SDP_BACKENDS``).  ``[b, h, s, d]`` in and out."""

    def __init__(self, dropout: float = 0.0, causal: bool = False, sdp_backend: Optional[str] = None):
        super().__init__()
        self.dropout, self.causal, self.sdp_backend = dropout, causal, sdp_backend

    def forward(self, q, k, v):
        return scaled_dot_product(q, k, v, self.sdp_backend, self.dropout if self.training else 0.0, self.causal)


class MultiHeadAttention(nn.Module):
    """q/k/v/output projections around an attention core; ``num_kv_heads < num_heads`` gives
    grouped-query attention.  ``sdp_backend="naive"`` selects the written-out core."""

    def __init__(self, hidden_dim: int, num_heads: int, dropout: float = 0.0, causal: bool = False, sdp_backend: Optional[str] = None, num_kv_heads: Optional[int] = None):
        super().__init__()
        assert hidden_dim % num_heads == 0
        self.h, self.kv = num_heads, num_kv_heads or num_heads
        assert self.h % self.kv == 0
        self.hd = hidden_dim // num_heads
        self.q = nn.Linear(hidden_dim, self.h * self.hd)
        self.k, self.v = nn.Linear(hidden_dim, self.kv * self.hd), nn.Linear(hidden_dim, self.kv * self.hd)
        self.proj = nn.Linear(hidden_dim, hidden_dim)
        self.core = Attention(dropout, causal) if sdp_backend == "naive" else FastAttention(dropout, causal, sdp_backend)

    def forward(self, x):
        b, s_, d = x.shape
        q = self.q(x).view(b, s_, self.h, self.hd).transpose(1, 2)
        k = self.k(x).view(b, s_, self.kv, self.hd).transpose(1, 2)
        v = self.v(x).view(b, s_, self.kv, self.hd).transpose(1, 2)
        if isinstance(self.core, Attention) and self.kv != self.h:
            k, v = k.repeat_interleave(self.h // self.kv, 1), v.repeat_interleave(self.h // self.kv, 1)
        return self.proj(self.core(q, k, v).transpose(1, 2).reshape(b, s_, d))


class SimpleAttention(nn.Module, _SampleMixin):
    """One head, no output projection, float inputs ``[b, 64, hidden]``."""

    seq_len = 64

    def __init__(self, hidden_dim: int, sdp_backend: Optional[str] = "naive"):
        super().__init__()
        self.hidden_dim = hidden_dim
        self.query, self.key, self.value = (nn.Linear(hidden_dim, hidden_dim, bias=False) for _ in range(3))
        self.core = Attention() if sdp_backend == "naive" else FastAttention(sdp_backend=sdp_backend)

    def forward(self, x):
        return self.core(self.query(x).unsqueeze(1), self.key(x).unsqueeze(1), self.value(x).unsqueeze(1)).squeeze(1)

    def get_sample(self, batch_size, dtype=torch.float32, device="cpu"):
        return torch.randn(batch_size, self.seq_len, self.hidden_dim, dtype=dtype, device=device)


class SimpleFastAttention(SimpleAttention):
    def __init__(self, hidden_dim: int, sdp_backend: Optional[str] = "FLASH_ATTENTION"):
        super().__init__(hidden_dim, sdp_backend)


class SimpleTransformer(nn.Module):
    """Embedding, ``n_blocks`` x (single-head attention, LayerNorm, GELU FFN, LayerNorm), head -
    no residual connections, the smallest thing that looks like a transformer to a partitioner."""

    def __init__(self, input_dim: int, hidden_dim: int, n_blocks: int = 4, seq_len: int = 64, ffn_dim: Optional[int] = None, sdp_backend: Optional[str] = "naive"):
        super().__init__()
        self.input_dim, self.hidden_dim, self.seq_len = input_dim, hidden_dim, seq_len
        self.embed = nn.Embedding(input_dim, hidden_dim)
        self.blocks = nn.Sequential(*[
            nn.Sequential(SimpleAttention(hidden_dim, sdp_backend), nn.LayerNorm(hidden_dim), FeedForward(hidden_dim, ffn_dim or 4 * hidden_dim), nn.LayerNorm(hidden_dim))
            for _ in range(n_blocks)
        ])
        self.head = nn.Linear(hidden_dim, input_dim, bias=False)

    def forward(self, ids):
        return self.head(self.blocks(self.embed(ids)))

    def get_sample(self, batch_size, dtype=None, device="cpu"):
        return torch.randint(0, self.input_dim, (batch_size, self.seq_len), device=device)

    get_target = get_sample

    @staticmethod
    def loss_fn(out, target, reduction="mean"):
        return F.cross_entropy(out.float().reshape(-1, out.size(-1)), target.reshape(-1), reduction=reduction)


class TransformerBlock(nn.Module):
    def __init__(self, hidden_dim: int, num_heads: int, ffn_dim: int, dropout: float = 0.0, causal: bool = False, sdp_backend: Optional[str] = None, num_kv_heads: Optional[int] = None):
        super().__init__()
        self.ln1, self.ln2 = nn.LayerNorm(hidden_dim), nn.LayerNorm(hidden_dim)
        self.attn = MultiHeadAttention(hidden_dim, num_heads, dropout, causal, sdp_backend, num_kv_heads)
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

    def __init__(self, input_dim: int = 1024, hidden_dim: int = 256, n_blocks: int = 4, seq_len: int = 128, num_heads: int = 4, ffn_dim: Optional[int] = None, dropout: float = 0.0, causal: bool = True, sdp_backend: Optional[str] = None, num_kv_heads: Optional[int] = None, **_unused):
        super().__init__()
        self.vocab, self.seq_len = input_dim, seq_len
        self.embed = TokenEmbedding(input_dim, hidden_dim, seq_len)
        self.blocks = nn.Sequential(*[TransformerBlock(hidden_dim, num_heads, ffn_dim or 4 * hidden_dim, dropout, causal, sdp_backend, num_kv_heads) for _ in range(n_blocks)])
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

    def __init__(self, hidden_dim: int = 256, n_blocks: int = 4, seq_len: int = 128, num_heads: int = 4, ffn_dim: Optional[int] = None, dropout: float = 0.0, sdp_backend: Optional[str] = None, num_kv_heads: Optional[int] = None, **_unused):
        super().__init__()
        self.hidden_dim, self.seq_len = hidden_dim, seq_len
        self.blocks = nn.Sequential(*[TransformerBlock(hidden_dim, num_heads, ffn_dim or 4 * hidden_dim, dropout, False, sdp_backend, num_kv_heads) for _ in range(n_blocks)])

    def forward(self, x):
        return self.blocks(x)

    def get_sample(self, batch_size, dtype=torch.float32, device="cpu"):
        return torch.randn(batch_size, self.seq_len, self.hidden_dim, dtype=dtype, device=device)


def make_simple_fno(fno_class):
    """Wrap a ``neuralop`` operator class (``FNO``, ``TFNO``) so that it offers ``get_sample`` /
    ``get_target`` / ``loss_fn`` like the rest of the zoo.  ``neuralop`` is optional: import it
    yourself and pass the class, e.g. ``SimpleFNO = make_simple_fno(neuralop.models.FNO)``."""

    class SimpleFNO(fno_class, _SampleMixin):
        def __init__(self, n_modes=(16, 16), hidden_channels: int = 32, in_channels: int = 3, out_channels: int = 3, resolution: int = 64, **kw):
            super().__init__(n_modes=n_modes, hidden_channels=hidden_channels, in_channels=in_channels, out_channels=out_channels, **kw)
            self._in, self._out, self._res, self._dims = in_channels, out_channels, resolution, len(n_modes)

        def get_sample(self, batch_size, dtype=torch.float32, device="cpu"):
            return torch.randn(batch_size, self._in, *([self._res] * self._dims), dtype=dtype, device=device)

        def get_target(self, batch_size, dtype=torch.float32, device="cpu"):
            return torch.randn(batch_size, self._out, *([self._res] * self._dims), dtype=dtype, device=device)

    SimpleFNO.__name__ = f"Simple{fno_class.__name__}"
    return SimpleFNO
