"""The engine's memory features on a GPU: rematerialisation options, activation offload through
the pinned arena and side streams, ILP profiling with CUDA events, `memory_budget`, timing and
memory statistics.  Single process, one GPU; numerics against the same model run plainly."""

import copy
import os

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def dev():
    from elf_b200.ops import _ext

    assert _ext.available(), "the native extension must be built for GPU tests"
    return torch.device("cuda", 0)


def _gpt(dev, scheduler, placement, with_sample=False, **kw):
    from elf_b200 import Pipeline, replace_layer_with_layer_dw
    from elf_b200.models.gpt import GPT, GPTConfig, gpt_stages

    cfg = GPTConfig(n_layers=2, d_model=128, n_heads=2, ffn=256, vocab=256, seq_len=64)
    torch.manual_seed(0)
    model = GPT(cfg).to(dev)
    ref = copy.deepcopy(model)
    stages = gpt_stages(model, len(placement))
    for s in stages:
        replace_layer_with_layer_dw(s)
    g = torch.Generator().manual_seed(1)
    tok = torch.randint(0, cfg.vocab, (4, cfg.seq_len + 1), generator=g).to(dev)
    ids, tgt = tok[:, :-1].contiguous(), tok[:, 1:].contiguous()
    pipe = Pipeline(stages, ids[:1] if with_sample else None, partitioner=False, scheduler=scheduler, placement=placement, outputs="device", **kw)
    return pipe, ref, GPT, ids, tgt


def _check(pipe, ref, GPT, ids, tgt, loss):
    rl = GPT.loss_fn(ref(ids), tgt)
    rl.backward()
    torch.testing.assert_close(loss, rl.detach(), atol=2e-4, rtol=2e-4)
    got = [p.grad for b in pipe.blocks for p in b.model.parameters()]
    want = [p.grad for p in ref.parameters()]
    assert len(got) == len(want)
    for a, b in zip(got, want):
        torch.testing.assert_close(a, b, atol=2e-4, rtol=2e-3)


def _solution(n_stages, nmb, **tables):
    zero = [[0] * nmb for _ in range(n_stages)]
    sol = {"objective": 0.0, "full_fwd": copy.deepcopy(zero), "activations_bwd": copy.deepcopy(zero), "full_bwd": copy.deepcopy(zero), "offload": copy.deepcopy(zero)}
    for name, cells in tables.items():
        for s, j in cells:
            sol[name][s][j] = 1
    return sol


@pytest.mark.parametrize(
    "tables",
    [
        dict(full_fwd=[(0, 0), (1, 1)], activations_bwd=[(0, 1), (1, 2)], full_bwd=[(1, 0)]),
        dict(offload=[(0, 0), (0, 2), (1, 1), (1, 3)]),
        dict(full_fwd=[(0, 1)], activations_bwd=[(1, 2)], full_bwd=[(1, 0)], offload=[(0, 2), (1, 3)]),
    ],
)
@pytest.mark.parametrize("base", ["1f1b", "zbv"])
def test_remat_and_offload_options_on_gpu(dev, tables, base):
    """Every (stage, micro-batch) option of the ILP's solution space, offload included (D2H on a
    side stream into the pinned arena, prefetch before the backward), leaves the numbers alone."""
    from elf_b200.registry import SCHEDULERS
    from elf_b200.scheduling.ilp import RematScheduler

    placement, nmb = [0, 0], 4
    sched = RematScheduler(SCHEDULERS[base], _solution(2, nmb, **tables))
    pipe, ref, GPT, ids, tgt = _gpt(dev, sched, placement)
    for _ in range(2):  # the second step reuses the arena's blocks
        pipe.zero_grad()
        _, loss = pipe(ids, tgt, GPT.loss_fn, split_size=1)
    torch.cuda.synchronize()
    _check(pipe, ref, GPT, ids, tgt, loss)


def test_offload_hooks_move_bytes_and_restore_them(dev):
    from elf_b200.execution.offload import OffloadToCPU, PinnedHostTensorPool

    pool = PinnedHostTensorPool(8 << 20)
    off = OffloadToCPU(pool=pool, min_bytes=1024)
    w = torch.randn(256, 256, device=dev, requires_grad=True)
    x = torch.randn(512, 256, device=dev, requires_grad=True)
    with off:
        h = x @ w
        y = (h * h).sum() + (h.t() * 2).sum()
    assert off.offloaded_bytes >= h.numel() * 4
    off.prefetch()
    y.backward()
    xr, wr = x.detach().clone().requires_grad_(), w.detach().clone().requires_grad_()
    hr = xr @ wr
    ((hr * hr).sum() + (hr.t() * 2).sum()).backward()
    torch.cuda.synchronize()
    torch.testing.assert_close(x.grad, xr.grad, atol=1e-3, rtol=1e-4)
    torch.testing.assert_close(w.grad, wr.grad, atol=1e-3, rtol=1e-4)
    off.release()
    assert pool.in_use == 0


def test_ilp_profile_solve_and_train_on_gpu(dev):
    """Profile the stages with CUDA events, tighten the budget until the solver rematerialises,
    train with that schedule, then let `memory_budget=` drive the same machinery."""
    from elf_b200.registry import SCHEDULERS
    from elf_b200.scheduling.ilp import profile_all_stages, solve_remat, stagerematify

    placement, nmb = [0, 0], 4
    pipe, ref, GPT, ids, tgt = _gpt(dev, "zbv", placement)
    stats = profile_all_stages(pipe.blocks, pipe.signatures, pipe.placement, ids[:1], None)
    assert len(stats) == 2 and all(st["T"]["f"] > 0 and st["M"]["f"] > 0 and st["Mparams"] > 0 for st in stats)
    free = solve_remat(stats, placement, SCHEDULERS["zbv"], nmb, 1e12, time_limit=20)
    chosen = None
    for frac in (0.98, 0.95, 0.92, 0.88, 0.84, 0.8, 0.75, 0.7):
        budget = frac * max(free["peak_mems"])
        try:
            sol = solve_remat(stats, placement, SCHEDULERS["zbv"], nmb, budget, time_limit=20)
        except RuntimeError:
            break
        if sum(map(sum, sol["full_fwd"])) + sum(map(sum, sol["activations_bwd"])) + sum(map(sum, sol["full_bwd"])) > 0:
            chosen = budget
            break
    assert chosen is not None, "no budget made the solver choose a remat option"
    pipe2, ref2, GPT, ids, tgt = _gpt(dev, stagerematify("zbv", stats, chosen), placement)
    _, loss = pipe2(ids, tgt, GPT.loss_fn, split_size=1)
    _check(pipe2, ref2, GPT, ids, tgt, loss)

    pipe3, ref3, GPT, ids, tgt = _gpt(dev, "zbv", placement, with_sample=True, memory_budget=chosen)
    assert len(pipe3.get_profiling_statistics()) == 2
    _, loss = pipe3(ids, tgt, GPT.loss_fn, split_size=1)
    _check(pipe3, ref3, GPT, ids, tgt, loss)


def test_timing_and_memory_statistics_on_gpu(dev):
    os.environ["ELF_TIMINGS"] = "1"
    os.environ["ELF_MEMORY"] = "1"
    try:
        pipe, ref, GPT, ids, tgt = _gpt(dev, "zbh1", [0])
        pipe(ids, tgt, GPT.loss_fn, split_size=2)
        torch.cuda.synchronize()
        assert set(pipe.stats) == {"total", "idle", "start_idle", "end_idle", "bubble"}
        assert pipe.stats["total"] > 0 and pipe.stats["idle"] <= pipe.stats["total"]
        names = set(pipe.detailed_stats["all_events"])
        assert {"forward(0:0)", "backward_inputs(0:1)", "backward_params(0:0)", "loss_forward"} <= names
        assert pipe.detailed_stats["peak_memory"], "ELF_MEMORY records the peak per operation"
    finally:
        os.environ.pop("ELF_TIMINGS")
        os.environ.pop("ELF_MEMORY")


def test_two_tensor_stage_boundary_on_gpu(dev):
    """Llama stages cut after a gate/up block: the boundary carries the residual stream and the
    activation, the producing stage has two outputs whose gradients arrive together (one autograd
    traversal, so the attention function's backward runs once).  Two stages on one GPU, ZB-V."""
    from elf_b200 import Pipeline
    from elf_b200.models.llama import LlamaConfig, build_llama_stages, llama_loss_fn, llama_stage_signatures
    from elf_b200.ops import gemm as G

    cfg = LlamaConfig(n_layers=3, d_model=256, n_heads=4, n_kv_heads=2, ffn=512, vocab=512, seq_len=128, rope_theta=10000.0)
    placement = [0, 0]
    sigs = llama_stage_signatures(cfg, 2, placement, "thirds")
    assert sigs[0].noutputs == 2 and sigs[1].ninputs == 2, "this shape is meant to be cut after a gate/up block"
    stages = build_llama_stages(cfg, 2, device=dev, seed=5, placement=placement, split_layers="thirds")
    ref = build_llama_stages(cfg, 2, device=dev, seed=5, placement=placement, split_layers="thirds", split_backward=False)
    g = torch.Generator().manual_seed(2)
    tok = torch.randint(0, cfg.vocab, (4, cfg.seq_len + 1), generator=g).to(dev)
    ids, tgt = tok[:, :-1].contiguous(), tok[:, 1:].contiguous()
    pipe = Pipeline(stages, None, partitioner=False, scheduler="zbv", placement=placement, outputs="none", signatures=sigs)
    _, loss = pipe(ids, tgt, llama_loss_fn, split_size=1)
    x = ids
    for s in ref:
        x = s(*x) if isinstance(x, tuple) else s(x)
    ref_loss = llama_loss_fn(x, tgt)
    ref_loss.backward()
    torch.cuda.synchronize()
    G.check_status(dev)
    assert abs(loss.item() - ref_loss.item()) < 2e-2 * abs(ref_loss.item())
    for block in pipe.blocks:
        want = {n: p.grad for n, p in ref[block.id].named_parameters()}
        for n, p in block.model.named_parameters():
            key = n if n in want else n.replace(".layer.", ".")
            err = ((p.grad.float() - want[key].float()).norm() / want[key].float().norm().clamp_min(1e-9)).item()
            assert err < 5e-2, (block.id, n, err)


def test_measured_cost_model_on_the_device(dev):
    """Timing the parts of a (small) layer on the GPU gives a usable cost model: shares of a layer
    add up to one, every part takes time, the head costs more than a norm would."""
    from elf_b200.models.llama import LlamaConfig, choose_llama_cut, llama_stage_costs
    from elf_b200.models.llama_costs import measure_cost_model

    cfg = LlamaConfig(n_layers=8, d_model=512, n_heads=4, n_kv_heads=2, ffn=1536, vocab=4096, seq_len=512, rope_theta=500000.0)
    cm = measure_cost_model(cfg, dev, mb_size=2, iters=2, burn_in_s=0.05)
    assert cm.source == "measured" and cm.layer_ms > 0
    assert abs(cm.attention + cm.mlp_up + cm.mlp_down - 1.0) < 1e-6
    assert min(cm.attention, cm.mlp_up, cm.mlp_down, cm.head, cm.embed) > 0
    assert abs(sum(cm.fbw) - 1.0) < 1e-6 and min(cm.fbw) > 0.0
    placement = [0, 1, 1, 0]
    mode = choose_llama_cut(cfg, 4, placement, cm)
    costs = llama_stage_costs(cfg, 4, placement, mode, cm)
    assert abs(sum(costs) - (cfg.n_layers + cm.head + cm.embed)) < 1e-6


def test_stream_order_checker_accepts_the_runtime_and_catches_a_missing_wait(dev):
    """With the stream-order debug mode on, a step that offloads activations, prefetches them and
    copies its outputs to the host raises nothing (every hand-off between streams is preceded by a
    wait); a hand-off made without the wait is reported."""
    from elf_b200.registry import SCHEDULERS
    from elf_b200.scheduling.ilp import RematScheduler
    from elf_b200.utils import stream_debug as sd

    sd.enable(True)
    try:
        placement, nmb = [0, 0], 4
        sched = RematScheduler(SCHEDULERS["1f1b"], _solution(2, nmb, offload=[(0, 0), (0, 2), (1, 1), (1, 3)]))
        pipe, ref, GPT, ids, tgt = _gpt(dev, sched, placement)
        pipe.engine.outputs = "cpu"
        out, loss = pipe(ids, tgt, GPT.loss_fn, split_size=1)
        torch.cuda.synchronize()
        assert len(out) == nmb and out[0].device.type == "cpu"
        # the same kind of hand-off without its wait
        side = torch.cuda.Stream(dev)
        buf = torch.ones(1 << 20, device=dev)
        sd.note_write(buf, torch.cuda.current_stream(dev), "compute result")
        with pytest.raises(sd.StreamOrderError):
            sd.check_read(buf, side, "side-stream copy")
        side.wait_stream(torch.cuda.current_stream(dev))
        sd.note_sync(side, torch.cuda.current_stream(dev))
        sd.check_read(buf, side, "side-stream copy")
    finally:
        sd.enable(False)
