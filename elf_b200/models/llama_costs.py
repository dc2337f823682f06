"""What the parts of a Llama-style decoder cost, for cutting it into pipeline stages.

The stage cut (``elf_b200.models.llama.half_layer_ranges``) balances the *time* per rank, so
it needs the time of an attention half, an MLP half (or its two parts), the embedding and the
LM head + loss, relative to a whole layer.  ``analytic_cost_model`` gives constants measured
once on the Llama-3-8B shape; ``measure_cost_model`` times the real blocks - forward,
input-gradient and weight-gradient passes, the way a pipeline stage runs them - on the device
the model will train on, which is what the reference's graph partitioners do per traced node
(``elf/partitioners/profile.py:75-96``).  Other shapes (1.3B, 13B, 70B) and other GPUs then get
a cut made for them instead of for the 8B shape.
"""

from __future__ import annotations

from dataclasses import asdict, dataclass
from typing import Dict, Optional, Tuple

import torch

__all__ = ["LlamaCostModel", "analytic_cost_model", "measure_cost_model"]


@dataclass
class LlamaCostModel:
    """Times in units of one whole decoder layer (forward + both backward passes).

    ``attention``   attention half (norm, QKV, RoPE, attention, output projection)
    ``mlp_up``      norm, gate/up projection, SwiGLU
    ``mlp_down``    down projection and residual add          (``attention + mlp_up + mlp_down = 1``)
    ``head``        final norm, vocabulary projection, loss
    ``embed``       embedding lookup and its gradient
    ``layer_ms``    milliseconds of one layer per micro-batch when measured, else ``None``
    ``fbw``         share of a layer's time spent in forward / input-gradient / weight-gradient passes
    ``micro_batches``  when set, the cut on a V placement is skewed for the pipeline's fill: rank ``r``
                    starts ``r`` forward stages late once per step, so it gets that much less work
    """

    attention: float
    mlp_up: float
    mlp_down: float
    head: float
    embed: float = 0.0
    layer_ms: Optional[float] = None
    fbw: Tuple[float, float, float] = (0.31, 0.44, 0.25)
    source: str = "analytic"
    micro_batches: Optional[int] = None

    @property
    def mlp(self) -> float:
        return self.mlp_up + self.mlp_down

    def shares(self, parts_per_layer: int) -> Tuple[float, ...]:
        """Relative cost of the 2 (attention, MLP) or 3 (attention, gate/up, down) parts of a layer."""
        return (self.attention, self.mlp) if parts_per_layer == 2 else (self.attention, self.mlp_up, self.mlp_down)

    def to_dict(self) -> Dict:
        return asdict(self)

    @staticmethod
    def from_dict(d: Dict) -> "LlamaCostModel":
        d = dict(d)
        d["fbw"] = tuple(d.get("fbw", (0.31, 0.44, 0.25)))
        return LlamaCostModel(**d)


def analytic_cost_model(cfg) -> LlamaCostModel:
    """Constants measured on B200 for the Llama-3-8B shape, scaled by FLOPs where a shape differs:
    the attention half takes 20 % of a layer, gate/up + SwiGLU 55 %, the down projection 25 %; the
    head's GEMMs run closer to the tensor-core peak than a layer's mix of GEMMs and bandwidth-bound
    kernels, so it costs 0.65 of what its FLOP count suggests."""
    d, hd = cfg.d_model, cfg.head_dim
    layer_flops = 2 * d * (cfg.n_heads + 2 * cfg.n_kv_heads) * hd + 2 * d * d + 6 * d * cfg.ffn + 2 * cfg.seq_len * d  # last term: causal attention
    head = 0.65 * 2 * d * cfg.vocab / layer_flops
    return LlamaCostModel(attention=0.2, mlp_up=0.55, mlp_down=0.25, head=head, embed=0.05)


class _PartTimer:
    """Runs one module on one micro-batch the way ``PipelineBlock`` runs a stage - the split-backward
    layers stash their operands in the forward and the backward, and compute weight gradients in a
    pass of their own - with a CUDA event between the passes."""

    def __init__(self, module, make_input, loss=None):
        from ..zb_utils import LayerDW

        self.module, self.make_input, self.loss = module, make_input, loss
        self.layers = [m for m in module.modules() if isinstance(m, LayerDW)]
        self.marks = []

    def _clear(self):
        for layer in self.layers:
            layer.clear()

    def run(self, timed: bool = True) -> None:
        """Enqueue forward, input-gradient and weight-gradient pass; nothing waits for the device."""

        def mark():
            e = torch.cuda.Event(enable_timing=True)
            e.record()
            return e

        e0 = mark()
        self._clear()
        out = self.module(*self.make_input())
        for layer in self.layers:
            layer.move_last_computed("input", 0)
        e1 = mark()
        if self.loss is not None:
            self.loss(out).backward()
        else:
            outs = out if isinstance(out, tuple) else (out,)
            live = [o for o in outs if o.requires_grad]
            torch.autograd.backward(live, [torch.ones_like(o) for o in live])
        for layer in self.layers:
            layer.move_last_computed("grad_output", 0)
        e2 = mark()
        for layer in self.layers:
            slots = layer.ctx["grad_output"]
            if slots and slots[0] is not None:
                layer.backward(0)
        e3 = mark()
        if timed:
            self.marks.append((e0, e1, e2, e3))

    def result(self) -> Tuple[float, float, float]:
        """Median (forward, input-gradient, weight-gradient) milliseconds of the timed runs; call
        after a device synchronisation."""

        def median(k):
            times = sorted(m[k].elapsed_time(m[k + 1]) for m in self.marks)
            return times[len(times) // 2]

        out = (median(0), median(1), median(2) if self.layers else 0.0)
        self._clear()
        self.marks.clear()
        for p in self.module.parameters():
            p.grad = None
        return out


def measure_cost_model(cfg, device=None, dtype=torch.bfloat16, mb_size: int = 1, iters: int = 10, group=None, burn_in_s: float = 0.7) -> LlamaCostModel:
    """Time one attention half, one gate/up part, one down part, the embedding and the head + loss
    of ``cfg`` on ``device`` (a CUDA device) for one micro-batch of ``mb_size`` sequences.  With
    ``group`` (a process group), rank 0's measurement is broadcast so that every rank cuts the model
    identically.  Falls back to ``analytic_cost_model`` on CPU.  The parts are timed in turn, ``iters``
    rounds, on a device kept busy (``burn_in_s`` seconds of work first, no idle gaps between the
    timed passes), so the ratios are those of a power-limited GPU in the middle of a step."""
    import torch.distributed as dist

    from . import llama as L
    from ..zb_utils import replace_layer_with_layer_dw

    device = torch.device(device) if device is not None else (torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else torch.device("cpu"))
    if device.type != "cuda":
        return analytic_cost_model(cfg)
    distributed = group is not None or (dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1)
    leader = (not distributed) or dist.get_rank(group) == 0
    model: Optional[LlamaCostModel] = None
    if leader:
        s, d = cfg.seq_len, cfg.d_model

        def build(cls):
            with torch.device(device):
                m = cls(cfg).to(dtype)
            L.init_llama_(m, cfg.init_std, 0)
            replace_layer_with_layer_dw(m)
            return m

        base = torch.randn(mb_size, s, d, device=device, dtype=dtype)
        act = torch.randn(mb_size, s, cfg.ffn, device=device, dtype=dtype)

        def hidden():
            return (base.detach().requires_grad_(True),)

        ids = torch.randint(0, cfg.vocab, (mb_size, s), device=device)
        target = torch.randint(0, cfg.vocab, (mb_size, s), device=device)
        jobs = {
            "mlp_up": (build(L.LlamaMLPUpBlock), hidden, None),
            "attention": (build(L.LlamaAttentionBlock), hidden, None),
            "mlp_down": (build(L.LlamaMLPDownBlock), lambda: (hidden()[0], act.detach().requires_grad_(True)), None),
            "embed": (build(L.LlamaEmbedding), lambda: (ids,), None),
            "head": (build(L.LlamaHead), hidden, lambda logits: L.llama_loss_fn(logits, target, reduction="sum")),
        }
        timers = {name: _PartTimer(*job) for name, job in jobs.items()}
        # Bring the device to the clock it sustains under load, then time the parts in turn,
        # round after round, with no host synchronisation until the end: the GPU stays loaded the
        # way it is inside a training step, and a drifting clock touches all parts alike.  (Timed
        # one pass at a time between synchronisations, the device idles in between and runs each
        # burst at a higher clock than its power limit lets it sustain; GEMM-heavy parts such as
        # the head then look cheaper, relative to a layer, than they are in a pipeline.)
        burner = timers["mlp_up"]
        burner.run(timed=False)  # first call: one-time set-up of the kernels
        burner.run()
        torch.cuda.synchronize(device)
        once = sum(burner.result())
        for _ in range(min(2000, int(1e3 * burn_in_s / once)) if once > 0 else 0):
            burner.run(timed=False)
        for i in range(1 + iters):
            for timer in timers.values():
                timer.run(timed=i > 0)
        torch.cuda.synchronize(device)
        t = {name: timer.result() for name, timer in timers.items()}
        del timers, burner
        del jobs
        torch.cuda.empty_cache()
        total = {k: sum(v) for k, v in t.items()}
        layer = total["attention"] + total["mlp_up"] + total["mlp_down"]
        parts = ("attention", "mlp_up", "mlp_down")
        fbw = tuple(sum(t[k][i] for k in parts) / layer for i in range(3))
        model = LlamaCostModel(
            attention=total["attention"] / layer,
            mlp_up=total["mlp_up"] / layer,
            mlp_down=total["mlp_down"] / layer,
            head=total["head"] / layer,
            embed=total["embed"] / layer,
            layer_ms=layer,
            fbw=fbw,
            source="measured",
        )
    if distributed:
        box = [model.to_dict() if model is not None else None]
        dist.broadcast_object_list(box, src=dist.get_global_rank(group, 0) if group is not None else 0, group=group)
        model = LlamaCostModel.from_dict(box[0])
    return model
