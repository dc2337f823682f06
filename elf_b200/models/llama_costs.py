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


def _time_ms(fn, iters: int, device) -> float:
    """Median device time of ``fn()`` over ``iters`` runs (CUDA events), after one untimed run."""
    fn()
    times = []
    for _ in range(iters):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        b.synchronize()
        times.append(a.elapsed_time(b))
    times.sort()
    return times[len(times) // 2]


def _fbw_of(module, make_input, device, iters: int, loss=None) -> Tuple[float, float, float]:
    """(forward, input-gradient, weight-gradient) milliseconds of one module on one micro-batch,
    run the way ``PipelineBlock`` runs a stage: the split-backward layers stash their operands in
    the forward and the backward, and compute weight gradients in a pass of their own."""
    from ..zb_utils import LayerDW

    layers = [m for m in module.modules() if isinstance(m, LayerDW)]
    state = {}

    def clear():
        for layer in layers:
            layer.clear()

    def forward():
        clear()
        args = make_input()
        state["in"] = args
        out = module(*args)
        state["out"] = out if not isinstance(out, tuple) else out
        for layer in layers:
            layer.move_last_computed("input", 0)

    def backward():
        forward_out = state["out"]
        if loss is not None:
            loss(forward_out).backward()
        else:
            outs = forward_out if isinstance(forward_out, tuple) else (forward_out,)
            live = [o for o in outs if o.requires_grad]
            torch.autograd.backward(live, [torch.ones_like(o) for o in live])
        for layer in layers:
            layer.move_last_computed("grad_output", 0)

    def weights():
        for layer in layers:
            slots = layer.ctx["grad_output"]
            if slots and slots[0] is not None:
                layer.backward(0)

    # each pass is timed on fresh state produced by untimed runs of the passes before it
    def timed(passes_before, the_pass):
        def run():
            for p in passes_before:
                p()
            torch.cuda.synchronize(device)

        times = []
        for i in range(iters + 1):
            run()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            the_pass()
            b.record()
            b.synchronize()
            if i:
                times.append(a.elapsed_time(b))
        times.sort()
        return times[len(times) // 2]

    f = timed([], forward)
    b = timed([forward], backward)
    w = timed([forward, backward], weights) if layers else 0.0
    clear()
    state.clear()
    for p in module.parameters():
        p.grad = None
    return f, b, w


def measure_cost_model(cfg, device=None, dtype=torch.bfloat16, mb_size: int = 1, iters: int = 3, group=None) -> LlamaCostModel:
    """Time one attention half, one gate/up part, one down part, the embedding and the head + loss
    of ``cfg`` on ``device`` (a CUDA device) for one micro-batch of ``mb_size`` sequences.  With
    ``group`` (a process group), rank 0's measurement is broadcast so that every rank cuts the model
    identically.  Falls back to ``analytic_cost_model`` on CPU."""
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

        def hidden():
            return (torch.randn(mb_size, s, d, device=device, dtype=dtype).requires_grad_(True),)

        t = {}
        t["attention"] = _fbw_of(build(L.LlamaAttentionBlock), hidden, device, iters)
        t["mlp_up"] = _fbw_of(build(L.LlamaMLPUpBlock), hidden, device, iters)
        t["mlp_down"] = _fbw_of(build(L.LlamaMLPDownBlock), lambda: (hidden()[0], torch.randn(mb_size, s, cfg.ffn, device=device, dtype=dtype).requires_grad_(True)), device, iters)
        ids = torch.randint(0, cfg.vocab, (mb_size, s), device=device)
        t["embed"] = _fbw_of(build(L.LlamaEmbedding), lambda: (ids,), device, iters)
        target = torch.randint(0, cfg.vocab, (mb_size, s), device=device)
        t["head"] = _fbw_of(build(L.LlamaHead), hidden, device, iters, loss=lambda logits: L.llama_loss_fn(logits, target, reduction="sum"))
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
