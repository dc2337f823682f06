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

import os

from dataclasses import dataclass
from typing import List, Optional, Sequence

import torch
import torch.nn as nn

from ..ops import attention as _attn
from ..ops import fused as _f
from . import llama_fused as _fused

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


# Whole layers / half layers as one autograd node each (see ``llama_fused``); ``ELF_B200_FUSED_LAYERS=0``
# keeps the chain of small autograd functions (numerics A/B, debugging).
FUSED_LAYERS = os.environ.get("ELF_B200_FUSED_LAYERS", "1") != "0"


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
        # the weight gradient is summed per token straight into the (flat) gradient buffer
        return _f.embedding(self.weight, ids, into_grad=True)


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

    fused = FUSED_LAYERS  # one autograd node with a hand-written backward (elf_b200.models.llama_fused)

    def forward(self, x):
        if self.fused and _fused.fused_apply(x, self.wqkv, self.wo, self.w_gate_up, self.w_down):
            return _fused.decoder_layer(self, x)
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


class LlamaAttentionBlock(nn.Module):
    """First half of a decoder layer (norm, QKV projection, RoPE, attention, output projection,
    residual add) as a module of its own, for stage boundaries that cut a layer in two."""

    _elf_leaf = True

    def __init__(self, cfg: LlamaConfig):
        super().__init__()
        d, hd = cfg.d_model, cfg.head_dim
        self.n_heads, self.n_kv_heads, self.head_dim, self.seq_len = cfg.n_heads, cfg.n_kv_heads, hd, cfg.seq_len
        self.theta = cfg.rope_theta
        self.norm1 = RMSNorm(d, cfg.eps)
        self.wqkv = nn.Linear(d, (cfg.n_heads + 2 * cfg.n_kv_heads) * hd, bias=False)
        self.wo = nn.Linear(cfg.n_heads * hd, d, bias=False)
        self._rope = None

    _tables = LlamaDecoderLayer._tables
    fused = FUSED_LAYERS

    def forward(self, x):
        if self.fused and _fused.fused_apply(x, self.wqkv, self.wo):
            return _fused.attention_half(self, x)
        b, s, d = x.shape
        hq, hkv, hd = self.n_heads, self.n_kv_heads, self.head_dim
        cos, sin = self._tables(x.device, s)
        qkv = self.wqkv(self.norm1(x).view(b * s, d))
        qkv = _f.rope_(qkv, cos, sin, hq + hkv, hd, s).view(b, s, hq + 2 * hkv, hd)
        a = _attn.attention_packed(qkv, hq, hkv, causal=True).reshape(b, s, hq * hd)
        return x + self.wo(a)


class LlamaMLPBlock(nn.Module):
    """Second half of a decoder layer (norm, gate/up projection, SwiGLU, down projection, residual add)."""

    _elf_leaf = True

    def __init__(self, cfg: LlamaConfig):
        super().__init__()
        d = cfg.d_model
        self.norm2 = RMSNorm(d, cfg.eps)
        self.w_gate_up = nn.Linear(d, 2 * cfg.ffn, bias=False)
        self.w_down = nn.Linear(cfg.ffn, d, bias=False)

    fused = FUSED_LAYERS

    def forward(self, x):
        if self.fused and _fused.fused_apply(x, self.w_gate_up, self.w_down):
            return _fused.mlp_half(self, x)
        return x + self.w_down(_f.swiglu(self.w_gate_up(self.norm2(x))))


class LlamaMLPUpBlock(nn.Module):
    """First part of the MLP half (norm, gate/up projection, SwiGLU).  Returns the residual stream
    and the activation: a stage boundary after this block carries two tensors."""

    _elf_leaf = True

    def __init__(self, cfg: LlamaConfig):
        super().__init__()
        self.norm2 = RMSNorm(cfg.d_model, cfg.eps)
        self.w_gate_up = nn.Linear(cfg.d_model, 2 * cfg.ffn, bias=False)

    def forward(self, x):
        return x, _f.swiglu(self.w_gate_up(self.norm2(x)))


class LlamaMLPDownBlock(nn.Module):
    """Second part of the MLP half: down projection of the activation added to the residual stream."""

    _elf_leaf = True

    def __init__(self, cfg: LlamaConfig):
        super().__init__()
        self.w_down = nn.Linear(cfg.ffn, cfg.d_model, bias=False)

    def forward(self, x, act):
        return x + self.w_down(act)


class LlamaHead(nn.Module):
    """Final norm + vocabulary projection.  With ``fused_loss`` the projection is left to the loss
    function (``elf_b200.ops.head_loss.ChunkedHeadLoss(head)``), which walks the vocabulary in chunks
    and never holds the logits: ``forward`` then returns the normalised hidden states."""

    _elf_leaf = True

    def __init__(self, cfg: LlamaConfig, fused_loss: bool = False):
        super().__init__()
        self.norm = RMSNorm(cfg.d_model, cfg.eps)
        self.out = nn.Linear(cfg.d_model, cfg.vocab, bias=False)
        self.fused_loss = fused_loss

    def forward(self, x):
        h = self.norm(x)
        return h if self.fused_loss else self.out(h)


class LlamaStage(nn.Sequential):
    """A contiguous run of the model: [embedding] + decoder layers (or parts of layers) + [head]."""


class LlamaTupleStage(LlamaStage):
    """A stage that holds a gate/up or a down block: a module that returns a tuple hands every
    element to the next module as its own argument, and the stage itself may take or return two
    tensors.  (A class of its own so that plain stages keep ``nn.Sequential``'s single-argument
    forward, which the graph tracers rely on.)"""

    def forward(self, *args):
        x = args if len(args) > 1 else args[0]
        for module in self:
            x = module(*x) if isinstance(x, tuple) else module(x)
        return x


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


# One big GEMM runs closer to the tensor-core peak than a decoder layer, whose time also goes into
# norms, RoPE, SwiGLU, attention and residual traffic: measured on B200 for the 8B shape, the
# head's three GEMMs + cross-entropy take 1.4-1.6 layer times where the FLOP ratio says 2.24.
HEAD_EFFICIENCY_VS_LAYER = 0.65


def head_cost_in_layers(cfg: LlamaConfig) -> float:
    """Time of the LM head (final norm + vocabulary projection + loss) in units of one decoder
    layer: the FLOP ratio scaled by how much more efficiently the head's GEMMs run."""
    d, hd = cfg.d_model, cfg.head_dim
    layer = 2 * d * (cfg.n_heads + 2 * cfg.n_kv_heads) * hd + 2 * d * d + 6 * d * cfg.ffn + 2 * cfg.seq_len * d  # last term: causal attention
    return HEAD_EFFICIENCY_VS_LAYER * 2 * d * cfg.vocab / layer


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


ATTENTION_SHARE = 0.2  # measured share of a decoder layer's forward+backward time spent in its attention half (8B shape, B200)


# (attention, gate/up + SwiGLU, down) shares of a layer's time when the MLP half is cut once more
THIRD_SHARES = (ATTENTION_SHARE, 0.55, 0.25)


def half_layer_ranges(n_layers: int, n_stages: int, placement: Optional[Sequence[int]] = None, head_units: float = 0.0, attention_share: float = ATTENTION_SHARE,
                      shares: Optional[Sequence[float]] = None, embed_units: float = 0.0, fill_share: float = 0.0):
    """Split the 2·n_layers half-layers (attention half, MLP half, attention half, ...) into
    ``n_stages`` contiguous ranges so that the busiest *rank* has as little work as possible.

    Whole layers cannot balance a pipeline whose last stage also carries the LM head: for the 8B
    shape on 8 ranks (V placement) the best whole-layer split gives two ranks 5 layers against a
    mean of 4.28 layer-units, a 14 % loss before any bubble.  With half-layers as the unit the
    busiest rank comes within a few percent of the mean.  Returns ``(ranges, costs)``:
    ``ranges[s] = (first, last+1)`` in half-layer indices, ``costs[s]`` in layer units (the head's
    ``head_units`` included in the last stage).  Local search from the proportional split:
    move one boundary by one half-layer while that lowers (max rank load, sum of squared loads).
    ``shares`` generalises the unit: a layer is cut into ``len(shares)`` consecutive parts of those
    relative costs (``THIRD_SHARES`` = attention, gate/up + SwiGLU, down projection) and the
    ranges index those parts.  ``embed_units`` is the cost of the embedding (in layers), carried
    by the first stage the way ``head_units`` is carried by the last.  ``fill_share`` (V placements):
    share of a stage's time that is its forward pass; rank ``r`` cannot start before the first
    micro-batch has gone through the ``r`` front stages before it, so that much is counted against
    its budget and ranks deep in the pipeline get correspondingly less work (all ranks then finish
    together instead of the last starter finishing last)."""
    shares = tuple(shares) if shares is not None else (attention_share, 1.0 - attention_share)
    k = len(shares)
    n_blocks = k * n_layers
    assert n_stages <= n_blocks, "more stages than layer parts"
    total_share = float(sum(shares))
    unit = [shares[b % k] / total_share for b in range(n_blocks)]
    unit[0] += embed_units  # the first layer part always sits in stage 0, next to the embedding
    prefix = [0.0]
    for u in unit:
        prefix.append(prefix[-1] + u)
    placement = list(placement) if placement is not None else list(range(n_stages))
    assert len(placement) == n_stages

    def stage_cost(bounds, s):
        return prefix[bounds[s + 1]] - prefix[bounds[s]] + (head_units if s == n_stages - 1 else 0.0)

    def score(bounds):
        load = {}
        for s in range(n_stages):
            load[placement[s]] = load.get(placement[s], 0.0) + stage_cost(bounds, s)
        return (round(max(load.values()), 9), round(sum(v * v for v in load.values()), 9))

    n_ranks = len(set(placement))
    is_v = n_stages == 2 * n_ranks and placement == list(range(n_ranks)) + list(range(n_ranks - 1, -1, -1))
    bounds = _v_bottleneck_bounds(prefix, n_ranks, head_units) if is_v else None
    if is_v and bounds is not None and fill_share > 0.0:
        # the offsets depend on the cut (time of the front stages before each rank): two rounds settle it
        for _ in range(3):
            fronts = [prefix[bounds[s + 1]] - prefix[bounds[s]] for s in range(n_ranks)]
            offsets, acc = [], 0.0
            for r in range(n_ranks):
                offsets.append(fill_share * acc)
                acc += fronts[r]
            # rank 0 runs the first forward and the last backward of a step and is never idle in
            # between: what it is given beyond its share delays everybody, so a margin is kept free
            # (measured on three 4- and 8-GPU boxes: its work ran 0.1, 0.3 and 0.5 layer units per
            # micro-batch over what the block times predicted - the loss, launch gaps, and a GPU
            # that never idles clocks lowest under the power limit)
            offsets[0] = FIRST_RANK_MARGIN
            again = _v_bottleneck_bounds(prefix, n_ranks, head_units, rank_offsets=offsets)
            if again is None or again == bounds:
                break
            bounds = again
        ranges = [(bounds[s], bounds[s + 1]) for s in range(n_stages)]
        return ranges, [stage_cost(bounds, s) for s in range(n_stages)]
    if bounds is None:
        # proportional start: stage s ends where the running cost reaches its share of the total
        # (the head's units count towards the last stages' share)
        total = prefix[-1] + head_units
        per_stage = [total / n_ranks / placement.count(placement[s]) for s in range(n_stages)]
        bounds, acc, b = [0], 0.0, 0
        for s in range(n_stages - 1):
            acc += per_stage[s]
            while b < n_blocks - (n_stages - 1 - s) and prefix[b + 1] <= acc + 1e-9:
                b += 1
            b = max(b, bounds[-1] + 1)
            bounds.append(b)
        bounds.append(n_blocks)
    # local search: shift a run of consecutive boundaries by one half-layer (a single boundary is
    # a run of one) while that lowers (max rank load, sum of squared loads)
    best = score(bounds)
    improved = True
    while improved:
        improved = False
        for i in range(1, n_stages):
            for k in range(i, n_stages):
                for step in (-1, 1):
                    trial = list(bounds)
                    for t in range(i, k + 1):
                        trial[t] += step
                    if any(trial[t] <= trial[t - 1] for t in range(1, n_stages + 1)):
                        continue
                    sc = score(trial)
                    if sc < best:
                        bounds, best, improved = trial, sc, True
    ranges = [(bounds[s], bounds[s + 1]) for s in range(n_stages)]
    return ranges, [stage_cost(bounds, s) for s in range(n_stages)]


THIRDS_GAIN = 0.02  # simulated gain below which a cut with three points per layer is not worth its two-tensor boundaries
FIRST_RANK_MARGIN = 0.3  # layer units per micro-batch kept free on rank 0 of a V placement when the cut allows for the pipeline's fill
BOTTLENECK_SLACK = 0.005  # partitions whose busiest rank is this close to the smallest possible one compete on the second criterion
LOAD_WEIGHT = 8.0  # weight of squared rank loads against squared stage costs when choosing among partitions within the bottleneck


def _v_bottleneck_bounds(prefix: List[float], n_ranks: int, head_units: float, window: float = 1.0, rank_offsets: Optional[Sequence[float]] = None) -> Optional[List[int]]:
    """Exact partition for the V placement ``[0..p-1, p-1..0]``: rank r owns the r-th range from
    the front and the r-th range from the back (the last one also carries the head).  First the
    smallest possible bottleneck T (busiest rank) is found by bisection; then, among the
    partitions whose ranks all stay within T, the one with the smallest sum of squared *stage*
    costs plus ``LOAD_WEIGHT`` times the sum of squared *rank* loads is taken.  The first term
    keeps a rank's two stages of similar size (a rank with a tiny front stage and a huge back
    stage is balanced on paper but lengthens the pipeline's fill and drain); the second keeps
    every rank, not only the busiest, close to the mean, so that a part whose cost was measured
    a few percent low does not turn a rank that sat just under T into the bottleneck (measured
    on 8 B200s: rank 0, which carries the head, was given 4.53 layer units under a T of 4.54
    and ran 4.8).  Both steps are a sweep over the ranks from the outside in over states
    (half-layers taken from the front, half-layers taken from the back)."""
    n, p = len(prefix) - 1, n_ranks
    if n < 2 * p:
        return None
    # rank_offsets[r]: time rank r cannot use anyway (it starts r hops after rank 0), counted
    # against its budget so that late starters get less work and all ranks finish together
    off = list(rank_offsets) if rank_offsets is not None else [0.0] * p

    def sweep(T, want_bounds, window=None):
        # states[(i, j)] = (sum of squared stage costs so far, previous state); with a window only
        # stages whose cost lies within `window` of T/2 are tried (the head counts for rank 0's back stage)
        states = {(0, n): (0.0, None)}
        trail = []
        for r in range(p):
            extra = head_units if r == 0 else 0.0
            left_after = 2 * (p - 1 - r)  # half-layers the remaining ranks need at least
            nxt = {}
            for (i, j), (sq, _) in states.items():
                for i2 in range(i + 1, j):
                    front = prefix[i2] - prefix[i]
                    budget = T - off[r] - extra - front
                    if budget < -1e-12:
                        break
                    if window is not None and (front < (T - off[r]) / 2 - window or front > (T - off[r]) / 2 + window):
                        continue
                    lo = i2 if r == p - 1 else i2 + left_after  # the last rank's back range closes the gap exactly
                    hi = i2 if r == p - 1 else j - 1
                    for j2 in range(hi, lo - 1, -1):
                        if j2 >= j:
                            continue
                        back = prefix[j] - prefix[j2]
                        if back > budget + 1e-12:
                            break
                        if window is not None and back + extra < (T - off[r]) / 2 - window:
                            continue
                        done = front + back + extra + off[r]
                        cand = sq + front * front + (back + extra) * (back + extra) + LOAD_WEIGHT * done * done
                        key = (i2, j2)
                        if key not in nxt or cand < nxt[key][0] - 1e-12:
                            nxt[key] = (cand, (i, j))
            if not nxt:
                return None
            trail.append(nxt)
            states = nxt
        ends = [(v[0], k) for k, v in states.items() if k[0] == k[1]]
        if not ends:
            return None
        if not want_bounds:
            return True
        _, key = min(ends)
        front, back = [], []
        for r in range(p - 1, -1, -1):
            front.append(key[0])
            back.append(key[1])
            key = trail[r][key][1]
        front.reverse()
        back.reverse()
        # boundaries: 0, the front ranges' ends, then the back ranges' starts from the innermost rank outwards, n
        return [0] + front + back[::-1][1:] + [n]

    def reachable(T):
        # feasibility only: for every front count keep the largest back count (smallest j) reachable
        reach = {0: n}
        for r in range(p):
            extra = head_units if r == 0 else 0.0
            left_after = 2 * (p - 1 - r)
            nxt = {}
            for i, j in reach.items():
                for i2 in range(i + 1, j):
                    budget = T - off[r] - extra - (prefix[i2] - prefix[i])
                    if budget < -1e-12:
                        break
                    if r == p - 1:
                        j2 = i2
                        if j2 >= j or prefix[j] - prefix[j2] > budget + 1e-12:
                            continue
                    else:
                        j2 = j - 1
                        if prefix[j] - prefix[j2] > budget + 1e-12:
                            continue
                        while j2 - 1 >= i2 + left_after and prefix[j] - prefix[j2 - 1] <= budget + 1e-12:
                            j2 -= 1
                        if j2 < i2 + left_after:
                            continue
                    if i2 not in nxt or j2 < nxt[i2]:
                        nxt[i2] = j2
            if not nxt:
                return False
            reach = nxt
        return any(j == i for i, j in reach.items())

    lo, hi = 0.0, prefix[-1] + head_units + max(off)
    if not reachable(hi):
        return None
    for _ in range(30):
        mid = 0.5 * (lo + hi)
        if reachable(mid):
            hi = mid
        else:
            lo = mid
    # 0.5 % of slack over the smallest bottleneck: costs are measured to a few percent, and the
    # second criterion chooses better among more partitions than the exact minimum admits
    T = hi * (1.0 + BOTTLENECK_SLACK) + 1e-9
    while window < T:
        got = sweep(T, True, window)
        if got is not None:
            return got
        window *= 2.0
    return sweep(T, True)


def _modules_for_range(cfg: LlamaConfig, first: int, last: int, k: int = 2) -> List[nn.Module]:
    """Modules of the layer parts [first, last) (k parts per layer): whole layers, and a whole MLP
    half, stay one fused module where all of their parts are inside."""
    mods: List[nn.Module] = []
    b = first
    while b < last:
        part = b % k
        if part == 0 and b + k <= last:
            mods.append(LlamaDecoderLayer(cfg))
            b += k
        elif part == 0:
            mods.append(LlamaAttentionBlock(cfg))
            b += 1
        elif k == 2 or (part == 1 and b + 2 <= last):
            mods.append(LlamaMLPBlock(cfg))
            b += k - 1
        elif part == 1:
            mods.append(LlamaMLPUpBlock(cfg))
            b += 1
        else:
            mods.append(LlamaMLPDownBlock(cfg))
            b += 1
    return mods


def _stage_ranges(cfg: LlamaConfig, n_stages: int, placement, split_layers, cost_model=None):
    """(ranges, parts per layer, costs) for ``split_layers`` = False, True / "halves" or "thirds".
    ``cost_model`` (``elf_b200.models.llama_costs.LlamaCostModel``) replaces the built-in constants
    for the parts of a layer, the head and the embedding - typically measured on the device."""
    fill = 0.0
    if cost_model is None:
        head = head_cost_in_layers(cfg) if placement is not None else 0.0
        embed, halves, thirds = 0.0, None, THIRD_SHARES
    else:
        head = cost_model.head if placement is not None else 0.0
        embed = cost_model.embed if placement is not None else 0.0
        halves, thirds = cost_model.shares(2), cost_model.shares(3)
        # a rank's wait for the first micro-batch happens once per step, its load once per micro-batch
        nmb = getattr(cost_model, "micro_batches", None)
        fill = float(cost_model.fbw[0]) / nmb if nmb else 0.0
    if split_layers in (True, "halves"):
        ranges, costs = half_layer_ranges(cfg.n_layers, n_stages, placement, head, shares=halves, embed_units=embed, fill_share=fill)
        return ranges, 2, costs
    if split_layers == "thirds":
        ranges, costs = half_layer_ranges(cfg.n_layers, n_stages, placement, head, shares=thirds, embed_units=embed, fill_share=fill)
        return ranges, 3, costs
    assert not split_layers, f"split_layers must be False, True, 'halves' or 'thirds', got {split_layers!r}"
    counts = layers_per_stage(cfg.n_layers, n_stages, placement, head)
    ends = [2 * sum(counts[: i + 1]) for i in range(n_stages)]
    ranges = [(ends[i] - 2 * counts[i], ends[i]) for i in range(n_stages)]
    head_last = head if placement is not None else head_cost_in_layers(cfg)
    return ranges, 2, [c + (head_last if i == n_stages - 1 else 0.0) + (embed if i == 0 else 0.0) for i, c in enumerate(counts)]


def _simulated_step(cfg: LlamaConfig, n_stages: int, placement: Sequence[int], mode, cost_model) -> float:
    """Length (in layer units) of one ZB-V step over the stages ``mode`` cuts, as the timeline
    simulator sees it: every stage's cost split into forward / input-gradient / weight-gradient
    passes by ``cost_model.fbw``, rank 0's margin counted as work."""
    from ..scheduling.scheduling import OperationType
    from ..scheduling.schedulers import generate_zbv_schedule
    from ..scheduling.simulator import simulate

    costs = list(_stage_ranges(cfg, n_stages, list(placement), mode, cost_model)[2])
    costs[0] += FIRST_RANK_MARGIN
    fbw = tuple(float(x) for x in cost_model.fbw)
    triples = [tuple(c * share for share in fbw) for c in costs]
    which = {OperationType.FORWARD: 0, OperationType.BACKWARD_INPUTS: 1, OperationType.BACKWARD_PARAMS: 2}
    n_ranks = len(set(placement))
    sched = generate_zbv_schedule(list(placement), cost_model.micro_batches, cap="auto", cap_limit=6 * n_ranks, stage_costs=triples)
    return simulate(sched, list(placement), lambda op: triples[op.block_id][which[op.op]] if op.op in which else 0.0).makespan


def choose_llama_cut(cfg: LlamaConfig, n_stages: int, placement: Sequence[int], cost_model=None, gain: float = 0.03):
    """``split_layers`` value to use for this placement: ``"thirds"`` (a third cut point per layer,
    after SwiGLU; that boundary carries two tensors) or ``True`` (cuts between attention and MLP
    halves only).  On a V placement with a cost model that knows the number of micro-batches, both
    cuts are laid out as ZB-V schedules and run through the timeline simulator, and thirds are taken
    when their step is at least ``THIRDS_GAIN`` (2 %) shorter: measured on 4 GPUs, a thirds cut whose
    simulated step was 1 % shorter ran no faster than the halves (780-789 ms against 774-791 ms),
    and its two-tensor boundaries cost memory for the second ring.  (The busiest rank's load alone misjudges it: on 8
    ranks with the Llama-3-8B shape the halves have the lighter busiest rank, 4.37 against 4.46
    layer units, but leave rank 0, which nothing can wait for, 2 % more work and the simulated and
    the measured step 4 % longer.)  Otherwise thirds are taken when they lower the busiest rank's
    load by more than ``gain``."""

    def busiest(mode):
        costs = _stage_ranges(cfg, n_stages, list(placement), mode, cost_model)[2]
        load = {}
        for s_, c in enumerate(costs):
            load[placement[s_]] = load.get(placement[s_], 0.0) + c
        return max(load.values())

    if n_stages > 3 * cfg.n_layers:
        return True
    n_ranks = len(set(placement))
    is_v = n_stages == 2 * n_ranks and list(placement) == list(range(n_ranks)) + list(range(n_ranks - 1, -1, -1))
    if is_v and n_ranks > 1 and cost_model is not None and getattr(cost_model, "micro_batches", None):
        return "thirds" if _simulated_step(cfg, n_stages, placement, "thirds", cost_model) < (1.0 - THIRDS_GAIN) * _simulated_step(cfg, n_stages, placement, True, cost_model) else True
    return "thirds" if busiest("thirds") < (1.0 - gain) * busiest(True) else True


def llama_stage_ranges(cfg: LlamaConfig, n_stages: int, placement: Optional[Sequence[int]] = None, split_layers=False, cost_model=None):
    """``(ranges, parts per layer, stage costs)`` of the cut ``build_llama_stages`` makes: ``ranges[s]`` is
    the half-open range of layer parts of stage ``s`` (2 parts per layer, 3 with ``"thirds"``)."""
    return _stage_ranges(cfg, n_stages, placement, split_layers, cost_model)


def llama_stage_signatures(cfg: LlamaConfig, n_stages: int, placement: Optional[Sequence[int]] = None, split_layers=False, cost_model=None):
    """Signatures of the stages ``build_llama_stages`` cuts: one tensor per boundary, except after a
    gate/up block (``split_layers="thirds"``), where the residual stream and the activation cross."""
    from ..partitioners.signature import Signature

    ranges, k, _ = _stage_ranges(cfg, n_stages, placement, split_layers, cost_model)
    width = [2 if (k == 3 and last % 3 == 2 and s != n_stages - 1) else 1 for s, (_, last) in enumerate(ranges)]  # tensors leaving stage s
    sigs = []
    for s in range(n_stages):
        n_in = 1 if s == 0 else width[s - 1]
        n_out = 1 if s == n_stages - 1 else width[s]
        ins = ["input"] if n_in == 1 else ["input", "input_act"]
        outs = ["output"] if n_out == 1 else ["output", "output_act"]
        sigs.append(Signature(ins, outs, [s - 1 if s else None] * n_in, [[s + 1 if s != n_stages - 1 else None]] * n_out))
    return sigs


def llama_stage_costs(cfg: LlamaConfig, n_stages: int, placement: Optional[Sequence[int]] = None, split_layers=False, cost_model=None) -> List[float]:
    """Cost of every stage in decoder-layer units (LM head and embedding included), as ``build_llama_stages`` cuts them."""
    return _stage_ranges(cfg, n_stages, placement, split_layers, cost_model)[2]


def build_llama_stages(cfg: LlamaConfig, n_stages: int, only: Optional[Sequence[int]] = None, device=None, dtype=torch.bfloat16, seed: int = 0, split_backward: bool = True, placement: Optional[Sequence[int]] = None, split_layers: bool = False, cost_model=None,
                       fused_head_loss: bool = False) -> List[Optional[LlamaStage]]:
    """Build the stages listed in ``only`` (all by default) directly on ``device``; the
    others are returned as ``None``, so a rank materialises only what it hosts.  Stage ``i``
    is seeded with ``seed + i``: the weights of a stage do not depend on who builds it.
    With ``placement`` the layer counts are balanced per rank (see ``layers_per_stage``);
    with ``split_layers`` a stage boundary may also fall between the attention half and the
    MLP half of a layer (see ``half_layer_ranges``), with ``split_layers="thirds"`` also after the
    MLP's SwiGLU, where two tensors cross the boundary (pass ``llama_stage_signatures(...)`` to the
    pipeline in that case).  ``cost_model`` (see ``elf_b200.models.llama_costs``) makes the cut for
    measured block times instead of the built-in constants; pass the same one to
    ``llama_stage_costs`` / ``llama_stage_signatures`` / ``llama_stage_ranges``.  With
    ``fused_head_loss`` the last stage ends with the final norm only and the vocabulary projection
    happens inside the loss (``elf_b200.ops.head_loss.ChunkedHeadLoss(stage[-1])`` as loss function)."""
    from ..zb_utils import replace_layer_with_layer_dw

    ranges, parts_per_layer, _ = _stage_ranges(cfg, n_stages, placement, split_layers, cost_model)
    stages: List[Optional[LlamaStage]] = []
    for i, (first, last) in enumerate(ranges):
        if only is not None and i not in only:
            stages.append(None)
            continue
        with torch.device(device if device is not None else "cpu"):
            mods: List[nn.Module] = []
            if i == 0:
                mods.append(LlamaEmbedding(cfg))
            mods += _modules_for_range(cfg, first, last, parts_per_layer)
            if i == n_stages - 1:
                mods.append(LlamaHead(cfg, fused_loss=fused_head_loss))
            tupled = any(isinstance(m, (LlamaMLPUpBlock, LlamaMLPDownBlock)) for m in mods)
            stage = (LlamaTupleStage if tupled else LlamaStage)(*mods).to(dtype)
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
