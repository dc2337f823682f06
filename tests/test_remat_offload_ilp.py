"""Rematerialisation options, activation offload, ILP and checkpointing through a
single-process pipeline on CPU (the same code paths run on GPUs)."""

import copy
import os

import pytest
import torch

from elf_b200 import Pipeline, replace_layer_with_layer_dw
from elf_b200.execution.offload import OffloadToCPU, PinnedHostTensorPool
from elf_b200.models.gpt import GPT, GPTConfig, gpt_stages
from elf_b200.registry import SCHEDULERS
from elf_b200.scheduling import OperationType, OpOptions, schedule_to_str
from elf_b200.scheduling.ilp import AutoScheduler, RematScheduler, profile_all_stages, solve_remat, stagerematify
from elf_b200.scheduling.offload_sched import offload_every

CFG = GPTConfig(n_layers=2, d_model=64, n_heads=2, ffn=128, vocab=128, seq_len=32)


def make(scheduler, placement, seed=0, **kw):
    torch.manual_seed(seed)
    model = GPT(CFG)
    ref = copy.deepcopy(model)
    stages = gpt_stages(model, len(placement))
    for s in stages:
        replace_layer_with_layer_dw(s)
    pipe = Pipeline(stages, None, partitioner=False, scheduler=scheduler, placement=placement, outputs="device", **kw)
    return pipe, ref


def data(batch=4):
    g = torch.Generator().manual_seed(1)
    tok = torch.randint(0, CFG.vocab, (batch, CFG.seq_len + 1), generator=g)
    return tok[:, :-1].contiguous(), tok[:, 1:].contiguous()


def check_against_reference(pipe, ref, ids, tgt, loss):
    rl = GPT.loss_fn(ref(ids), tgt)
    rl.backward()
    torch.testing.assert_close(loss, rl.detach(), atol=1e-4, rtol=1e-4)
    got = [p.grad for b in pipe.blocks for p in b.model.parameters()]
    want = [p.grad for p in ref.parameters()]
    assert len(got) == len(want)
    for a, b in zip(got, want):
        torch.testing.assert_close(a, b, atol=1e-4, rtol=1e-3)


def fixed_solution(n_stages, nmb, **tables):
    zero = [[0] * nmb for _ in range(n_stages)]
    sol = {"objective": 0.0, "full_fwd": copy.deepcopy(zero), "activations_bwd": copy.deepcopy(zero), "full_bwd": copy.deepcopy(zero), "offload": copy.deepcopy(zero)}
    for name, cells in tables.items():
        for s, j in cells:
            sol[name][s][j] = 1
    return sol


@pytest.mark.parametrize(
    "tables",
    [
        dict(full_fwd=[(0, 0), (1, 1), (0, 3)]),
        dict(activations_bwd=[(0, 1), (1, 0), (1, 3)]),
        dict(full_bwd=[(0, 0), (1, 2)]),
        dict(offload=[(0, 0), (0, 2), (1, 1)]),
        dict(full_fwd=[(0, 1)], activations_bwd=[(0, 1), (1, 2)], full_bwd=[(1, 0)], offload=[(0, 2)]),
    ],
)
@pytest.mark.parametrize("base", ["1f1b", "zbv"])
def test_every_remat_option_keeps_the_numbers(tables, base):
    placement = [0, 0]
    nmb = 4
    sched = RematScheduler(SCHEDULERS[base], fixed_solution(2, nmb, **tables))
    pipe, ref = make(sched, placement)
    ids, tgt = data()
    text = schedule_to_str(sched(placement, nmb))
    if "activations_bwd" in tables or "full_bwd" in tables:
        assert "R" in text
    if "offload" in tables:
        assert "P" in text
    _, loss = pipe(ids, tgt, GPT.loss_fn, split_size=1)
    check_against_reference(pipe, ref, ids, tgt, loss)


def test_whole_stage_checkpoint_scheduler():
    pipe, ref = make("full_remat", [0])
    ids, tgt = data()
    _, loss = pipe(ids, tgt, GPT.loss_fn, split_size=2)
    check_against_reference(pipe, ref, ids, tgt, loss)


def test_offload_wrapper_and_hooks():
    sched = offload_every("1f1b", 2, prefetching_time=1)([0, 1], 4)
    marked = [op for op in sched if op.options.get(OpOptions.ACTIVATION_OFFLOAD)]
    assert {op.mb_id for op in marked} == {0, 2}
    assert sum(op.op is OperationType.PREFETCH_ACTIVATIONS for op in sched) == 4
    for r in (0, 1):
        prog = [op for op in sched if op.rank == r]
        for i, op in enumerate(prog):
            if op.op is OperationType.PREFETCH_ACTIVATIONS:
                later_b = [j for j, o in enumerate(prog) if o.op is OperationType.BACKWARD_INPUTS and o.mb_id == op.mb_id and o.block_id == op.block_id]
                earlier_f = [j for j, o in enumerate(prog) if o.op is OperationType.FORWARD and o.mb_id == op.mb_id and o.block_id == op.block_id]
                assert earlier_f[0] < i < later_b[0]

    # the hook layer itself: views of one storage share one host copy; small tensors pass through
    pool = PinnedHostTensorPool(1 << 20)
    off = OffloadToCPU(pool=pool, min_bytes=1024)
    w = torch.randn(64, 64, requires_grad=True)
    x = torch.randn(128, 64, requires_grad=True)
    with off:
        h = x @ w
        y = (h * h).sum() + (h.t() * 2).sum() + (x[:1] * 3).sum()
    assert off.offloaded_bytes > 0
    off.prefetch()
    y.backward()
    xr, wr = x.detach().clone().requires_grad_(), w.detach().clone().requires_grad_()
    hr = xr @ wr
    ((hr * hr).sum() + (hr.t() * 2).sum() + (xr[:1] * 3).sum()).backward()
    torch.testing.assert_close(x.grad, xr.grad)
    torch.testing.assert_close(w.grad, wr.grad)
    off.release()
    assert pool.in_use == 0 and pool.size() >= 1 << 20


def test_pinned_pool_reuses_and_coalesces():
    pool = PinnedHostTensorPool(1 << 16)
    a = pool.allocate(1000, torch.float32)
    b = pool.allocate(3000, torch.bfloat16)
    assert a.dtype == torch.float32 and a.numel() == 1000 and b.numel() == 3000
    a.fill_(1.0)
    b.fill_(2.0)
    assert a.sum().item() == 1000
    cap = pool.size()
    pool.free(a)
    pool.free(b)
    c = pool.allocate(cap // 4, torch.float32)  # the whole first block again: holes were merged
    assert pool.size() == cap
    pool.free(c)
    pool.reserve(1 << 20)
    assert pool.size() >= 1 << 20


def test_ilp_profiles_solves_and_trains():
    placement = [0, 0]
    pipe, ref = make("zbv", placement)
    ids, tgt = data()
    stats = profile_all_stages(pipe.blocks, pipe.signatures, pipe.placement, ids[:1], None)
    assert len(stats) == 2
    for st in stats:
        for key in ("T", "M", "Mpeak", "Mpeak_ckpt", "Mparams", "Mba", "Mbg", "Minput", "Moutput", "Tcomm"):
            assert key in st
        assert st["T"]["f"] > 0 and st["M"]["f"] > 0 and st["Mba"] > 0
    nmb = 4
    free = solve_remat(stats, placement, SCHEDULERS["zbv"], nmb, 1e9, time_limit=20)
    assert sum(map(sum, free["full_fwd"])) + sum(map(sum, free["activations_bwd"])) + sum(map(sum, free["full_bwd"])) == 0
    n_options = lambda sol: sum(map(sum, sol["full_fwd"])) + sum(map(sum, sol["activations_bwd"])) + sum(map(sum, sol["full_bwd"]))
    tight, tight_budget = None, None
    for frac in (0.98, 0.95, 0.92, 0.88, 0.84, 0.8, 0.75):  # tighten until the solver has to rematerialise
        budget = frac * max(free["peak_mems"])
        try:
            sol = solve_remat(stats, placement, SCHEDULERS["zbv"], nmb, budget, time_limit=20)
        except RuntimeError:
            break
        if n_options(sol) > 0:
            tight, tight_budget = sol, budget
            break
    assert tight is not None, "no budget made the solver choose a remat option"
    assert max(tight["peak_mems"]) <= tight_budget + 1e-6
    assert tight["objective"] >= free["objective"] - 1e-6
    with pytest.raises(RuntimeError, match="infeasible"):
        solve_remat(stats, placement, SCHEDULERS["zbv"], nmb, 0.5 * sum(s["Mparams"] for s in stats), time_limit=10)
    # offload becomes attractive when the link is fast
    off = solve_remat(stats, placement, SCHEDULERS["zbv"], nmb, tight_budget, time_limit=20, offload=True, pcie_gbs=1e4)
    assert "offload" in off and off["objective"] <= tight["objective"] + 1e-6

    remat = stagerematify("zbv", stats, tight_budget)
    pipe2, ref2 = make(remat, placement)
    _, loss = pipe2(ids, tgt, GPT.loss_fn, split_size=1)
    check_against_reference(pipe2, ref2, ids, tgt, loss)
    assert remat.solution is not None

    auto = AutoScheduler(stats, tight_budget, time_limit=10)
    sched = auto(placement, nmb)
    assert auto.best[1] in SCHEDULERS and len(sched) > 0


def test_pipeline_memory_budget_end_to_end():
    torch.manual_seed(0)
    model = GPT(CFG)
    stages = gpt_stages(model, 2)
    for s in stages:
        replace_layer_with_layer_dw(s)
    ids, tgt = data()
    pipe = Pipeline(stages, ids[:1], partitioner=False, scheduler="zbv", placement=[0, 0], memory_budget=1e6, outputs="device")
    assert len(pipe.get_profiling_statistics()) == 2
    out, loss = pipe(ids, tgt, GPT.loss_fn, split_size=1)
    assert len(out) == 4 and torch.isfinite(loss)


def test_pipeline_offload_option_reaches_the_ilp(monkeypatch):
    """``Pipeline(memory_budget=..., offload=True)`` asks the solver for offload decisions."""
    import elf_b200.scheduling.ilp as ilp

    seen = {}
    real = ilp.solve_remat

    def spy(*args, **kwargs):
        seen.update(kwargs)
        return real(*args, **kwargs)

    monkeypatch.setattr(ilp, "solve_remat", spy)
    torch.manual_seed(0)
    stages = gpt_stages(GPT(CFG), 2)
    for s in stages:
        replace_layer_with_layer_dw(s)
    ids, tgt = data()
    pipe = Pipeline(stages, ids[:1], partitioner=False, scheduler="zbv", placement=[0, 0], memory_budget=1e6, offload=True, outputs="device")
    out, loss = pipe(ids, tgt, GPT.loss_fn, split_size=1)
    assert seen.get("offload") is True
    assert "offload" in pipe.scheduler.solution
    assert len(out) == 4 and torch.isfinite(loss)


def test_checkpoint_roundtrip(tmp_path):
    pipe, ref = make("1f1b", [0])
    path = pipe.checkpoint(epoch=3, dir_path=str(tmp_path), extra={"optimizer": {"step": 7}})
    assert path.endswith(os.path.join("3", "dp0_pp0.pt"))
    state = torch.load(path, weights_only=False)
    assert state["rank"] == 0 and state["pp"] == 0 and state["dp"] == 0 and state["epoch"] == 3
    assert set(state["state_dict_0"]) == set(pipe.blocks[0].model.state_dict())
    before = {k: v.clone() for k, v in pipe.blocks[0].model.state_dict().items()}
    with torch.no_grad():
        for p in pipe.parameters():
            p.add_(1.0)
    loaded = pipe.load_checkpoint(epoch=3, dir_path=str(tmp_path))
    assert loaded["optimizer"] == {"step": 7}
    for k, v in pipe.blocks[0].model.state_dict().items():
        torch.testing.assert_close(v, before[k])
    merged = pipe.gather_parameters()
    assert set(merged) == {n for n, _ in pipe.named_parameters()}
    pipe.save(str(tmp_path / "flat.pt"))
    flat = torch.load(str(tmp_path / "flat.pt"))
    assert set(flat) == set(merged)


def test_stats_and_inference():
    os.environ["ELF_TIMINGS"] = "1"
    try:
        pipe, _ = make("1f1b", [0])
        ids, tgt = data()
        pipe(ids, tgt, GPT.loss_fn, split_size=2)
        assert set(pipe.stats) == {"total", "idle", "start_idle", "end_idle", "bubble"}
        assert {"all_events", "memories", "peak_memory"} <= set(pipe.detailed_stats)
        names = set(pipe.detailed_stats["all_events"])
        assert {"forward(0:0)", "backward_inputs(0:1)", "backward_params(0:0)", "loss_forward", "backward(0:0)"} <= names
        assert pipe.stats["idle"] <= pipe.stats["total"]
    finally:
        os.environ.pop("ELF_TIMINGS")
    out, loss = pipe(ids, None, None, split_size=2, scheduler="inference")
    assert loss is None and len(out) == 2 and out[0].shape == (2, CFG.seq_len, CFG.vocab)
    pipe.zero_grad()
    assert all(p.grad is None for p in pipe.parameters())


def test_measured_stage_costs_needs_a_timed_step():
    pipe, _ = make("zbv", [0, 0])
    ids, tgt = data()
    pipe(ids, tgt, GPT.loss_fn, split_size=1)
    with pytest.raises(RuntimeError, match="ELF_TIMINGS"):
        pipe.measured_stage_costs()
    os.environ["ELF_TIMINGS"] = "1"
    try:
        pipe.zero_grad()
        pipe(ids, tgt, GPT.loss_fn, split_size=1)
    finally:
        os.environ.pop("ELF_TIMINGS")
    costs = pipe.measured_stage_costs()
    assert len(costs) == 2 and all(f > 0 and b > 0 and w > 0 for f, b, w in costs)
    pipe.set_scheduler("1f1b")
    pipe.zero_grad()
    _, loss = pipe(ids, tgt, GPT.loss_fn, split_size=1)
    assert torch.isfinite(loss)


def test_remat_options_with_a_two_tensor_stage_boundary():
    """Stages cut after a gate/up block (two outputs) under every rematerialisation option: the
    recompute-backward differentiates both outputs in one traversal."""
    from elf_b200.models.llama import LlamaConfig, build_llama_stages, llama_loss_fn, llama_stage_signatures

    cfg = LlamaConfig(n_layers=3, d_model=64, n_heads=4, n_kv_heads=2, ffn=128, vocab=512, seq_len=32, rope_theta=10000.0)
    placement, nmb = [0, 0], 4
    sigs = llama_stage_signatures(cfg, 2, placement, "thirds")
    assert sigs[0].noutputs == 2
    stages = build_llama_stages(cfg, 2, dtype=torch.float32, seed=5, placement=placement, split_layers="thirds")
    ref = build_llama_stages(cfg, 2, dtype=torch.float32, seed=5, placement=placement, split_layers="thirds", split_backward=False)
    sched = RematScheduler(SCHEDULERS["zbv"], fixed_solution(2, nmb, full_fwd=[(0, 1)], activations_bwd=[(0, 2), (1, 0)], full_bwd=[(0, 0), (1, 3)]))
    pipe = Pipeline(stages, None, partitioner=False, scheduler=sched, placement=placement, outputs="none", signatures=sigs)
    g = torch.Generator().manual_seed(2)
    tok = torch.randint(0, cfg.vocab, (4, cfg.seq_len + 1), generator=g)
    ids, tgt = tok[:, :-1].contiguous(), tok[:, 1:].contiguous()
    _, loss = pipe(ids, tgt, llama_loss_fn, split_size=1)
    x = ids
    for s in ref:
        x = s(*x) if isinstance(x, tuple) else s(x)
    ref_loss = llama_loss_fn(x, tgt)
    ref_loss.backward()
    torch.testing.assert_close(loss, ref_loss.detach(), atol=1e-4, rtol=1e-4)
    for block in pipe.blocks:
        want = {n: p.grad for n, p in ref[block.id].named_parameters()}
        for n, p in block.model.named_parameters():
            torch.testing.assert_close(p.grad, want[n if n in want else n.replace(".layer.", ".")], atol=1e-4, rtol=1e-3)
