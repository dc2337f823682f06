"""Stage cuts of the Llama-style decoder: cost models, where the boundaries fall, which
granularity is chosen."""

import pytest
import torch

from elf_b200.models.llama import LLAMA_CONFIGS, build_llama_stages, choose_llama_cut, llama_stage_costs, llama_stage_ranges, llama_stage_signatures
from elf_b200.models.llama_costs import LlamaCostModel, analytic_cost_model, measure_cost_model

CFG = LLAMA_CONFIGS["llama3-8b"]


def v(pp):
    return list(range(pp)) + list(range(pp - 1, -1, -1))


def loads(costs, placement):
    out = {}
    for s, c in enumerate(costs):
        out[placement[s]] = out.get(placement[s], 0.0) + c
    return [out[r] for r in sorted(out)]


def test_cost_model_roundtrip_and_cpu_fallback():
    cm = analytic_cost_model(CFG)
    assert abs(cm.attention + cm.mlp_up + cm.mlp_down - 1.0) < 1e-9 and cm.head > 1.0
    assert LlamaCostModel.from_dict(cm.to_dict()) == cm
    assert cm.shares(2) == (cm.attention, cm.mlp) and len(cm.shares(3)) == 3
    assert measure_cost_model(CFG, "cpu").source == "analytic"


def test_a_costlier_embedding_moves_work_off_the_first_rank():
    pl = v(8)
    light = LlamaCostModel(0.2, 0.55, 0.25, head=1.0, embed=0.0)
    heavy = LlamaCostModel(0.2, 0.55, 0.25, head=1.0, embed=0.8)
    r_light = llama_stage_ranges(CFG, 16, pl, "thirds", light)[0]
    r_heavy = llama_stage_ranges(CFG, 16, pl, "thirds", heavy)[0]
    parts = lambda r: (r[0][1] - r[0][0]) + (r[15][1] - r[15][0])  # layer parts on rank 0 (first and last stage)
    assert parts(r_heavy) < parts(r_light)
    for ranges in (r_light, r_heavy):  # contiguous cover of all 96 parts
        assert ranges[0][0] == 0 and ranges[-1][1] == 3 * CFG.n_layers
        assert all(a[1] == b[0] and a[1] > a[0] for a, b in zip(ranges, ranges[1:]))
    costs = llama_stage_costs(CFG, 16, pl, "thirds", heavy)
    assert abs(sum(costs) - (CFG.n_layers + 1.0 + 0.8)) < 1e-6
    ld = loads(costs, pl)
    assert max(ld) / (sum(ld) / len(ld)) < 1.05


def test_cut_granularity_follows_the_balance():
    cm = LlamaCostModel(0.2, 0.55, 0.25, head=1.0, embed=0.3)
    assert choose_llama_cut(CFG, 16, v(8), cm) == "thirds"  # halves leave one rank 10 % above the mean
    assert choose_llama_cut(CFG, 4, v(2), cm) is True  # two ranks balance with halves already
    # signatures and built stages agree with the chosen ranges
    small = LLAMA_CONFIGS["llama-tiny"]
    pl = v(2)
    mode = "thirds"
    sigs = llama_stage_signatures(small, 4, pl, mode, cm)
    stages = build_llama_stages(small, 4, device="cpu", dtype=torch.float32, placement=pl, split_layers=mode, cost_model=cm)
    x = torch.randint(0, small.vocab, (2, small.seq_len))
    out = (x,)
    for sig, stage in zip(sigs, stages):
        assert len(sig.inputs) == len(out)
        y = stage(*out)
        out = y if isinstance(y, tuple) else (y,)
        assert len(sig.outputs) == len(out)
    assert out[0].shape == (2, small.seq_len, small.vocab)


def test_cut_allows_for_the_pipeline_fill():
    """With the number of micro-batches known, ranks deep in a V pipeline (which start late, once per
    step) get less work: what is minimised is load + time lost waiting for the first micro-batch."""
    pl = v(8)
    base = LlamaCostModel(0.32, 0.45, 0.23, head=1.8, embed=0.04, fbw=(0.34, 0.42, 0.24))
    skew = LlamaCostModel(0.32, 0.45, 0.23, head=1.8, embed=0.04, fbw=(0.34, 0.42, 0.24), micro_batches=16)

    def finish(model):
        costs = llama_stage_costs(CFG, 16, pl, "thirds", model)
        ld = loads(costs, pl)
        fill = [0.34 / 16 * sum(costs[:r]) for r in range(8)]
        return max(a + b for a, b in zip(ld, fill)), ld

    t0, ld0 = finish(base)
    t1, ld1 = finish(skew)
    assert t1 < t0
    assert ld1[0] > ld1[-1] and sum(ld1) == pytest.approx(sum(ld0))


def test_cut_granularity_by_simulated_step_and_first_rank_margin():
    """With the number of micro-batches known, halves against thirds is decided by laying both cuts
    out as ZB-V and simulating the step; rank 0 is kept a little lighter than the busiest rank."""
    import elf_b200.models.llama as L

    cm = LlamaCostModel(attention=0.315, mlp_up=0.4625, mlp_down=0.2225, head=1.9, embed=0.024, layer_ms=5.6, fbw=(0.331, 0.409, 0.26), source="measured", micro_batches=16)
    pl = v(8)
    halves, thirds = L._simulated_step(CFG, 16, pl, True, cm), L._simulated_step(CFG, 16, pl, "thirds", cm)
    assert halves > 0 and thirds > 0
    expected = "thirds" if thirds < (1.0 - L.THIRDS_GAIN) * halves else True
    assert choose_llama_cut(CFG, 16, pl, cm) == expected
    assert choose_llama_cut(CFG, 16, pl, cm) == choose_llama_cut(CFG, 16, pl, LlamaCostModel.from_dict(cm.to_dict()))  # every rank decides alike
    for mode in (True, "thirds"):
        ld = loads(llama_stage_costs(CFG, 16, pl, mode, cm), pl)
        assert ld[0] <= max(ld[1:]) + 1e-9, ld  # rank 0 runs the head, the loss and the first and last operation of a step
        assert max(ld) / (sum(ld) / len(ld)) < 1.07  # the others carry what rank 0 is spared
    # without the number of micro-batches the rule of thumb (busiest rank) still answers
    cm.micro_batches = None
    assert choose_llama_cut(CFG, 16, pl, cm) in (True, "thirds")


def test_cuts_for_random_cost_models_cover_the_model():
    """Whatever the measured block times say, the cut is a contiguous cover of all layer parts, the
    stage costs add up, and the granularity choice answers."""
    import random

    rng = random.Random(2)
    done = 0
    while done < 12:
        cfg = LLAMA_CONFIGS[rng.choice(["llama3-8b", "llama-1.3b", "llama-13b", "llama-tiny"])]
        p = rng.choice((2, 4, 8))
        if 2 * p > 2 * cfg.n_layers:
            continue
        a, u = rng.uniform(0.15, 0.45), rng.uniform(0.3, 0.5)
        f = rng.uniform(0.25, 0.4)
        cm = LlamaCostModel(attention=a, mlp_up=u, mlp_down=1 - a - u, head=rng.uniform(0.3, 3.0), embed=rng.uniform(0, 0.3), layer_ms=rng.uniform(0.5, 10),
                            fbw=(f, 0.4, 0.6 - f), source="measured", micro_batches=rng.choice((None, 2 * p, 16)))
        pl = v(p)
        for mode in (True, "thirds"):
            ranges, k, costs = llama_stage_ranges(cfg, 2 * p, pl, mode, cm)
            assert ranges[0][0] == 0 and ranges[-1][1] == k * cfg.n_layers
            assert all(x[1] == y[0] and x[1] > x[0] for x, y in zip(ranges, ranges[1:]))
            assert abs(sum(costs) - (cfg.n_layers + cm.head + cm.embed)) < 1e-6
        assert choose_llama_cut(cfg, 2 * p, pl, cm) in (True, "thirds")
        done += 1
