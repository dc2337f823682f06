"""End-to-end numerics of the runtime on CPU/gloo ranks against the non-pipelined model."""

import copy

import pytest
import torch

from tests.dist_utils import run_ranks

pytestmark = pytest.mark.dist

ATOL = RTOL = 1e-3


def _reference(model, ids, targets, lr=1e-3):
    ref = copy.deepcopy(model)
    loss = ref.loss_fn(ref(ids), targets)
    loss.backward()
    grads = {n: p.grad.clone() for n, p in ref.named_parameters()}
    opt = torch.optim.AdamW(ref.parameters(), lr=lr)
    opt.step()
    return loss.detach(), grads, {n: p.detach().clone() for n, p in ref.named_parameters()}


def _stage_param_names(model, n_stages):
    """Map (stage, local name) -> global name for the flat sequential split."""
    from elf_b200.models.gpt import gpt_stages

    names = {}
    idx = 0
    for s, stage in enumerate(gpt_stages(model, n_stages)):
        for local_idx, layer in enumerate(stage.children()):
            for n, _ in layer.named_parameters():
                names[(s, f"{local_idx}.{n}")] = f"{idx}.{n}"
            idx += 1
    return names


def _worker(rank, world, scheduler, placement, dp, nmb, split_w, strict=False):
    import os

    if strict:
        os.environ["ELF_B200_P2P_STRICT"] = "1"
    from elf_b200 import Pipeline, replace_layer_with_layer_dw
    from elf_b200.models.gpt import GPT, GPTConfig, gpt_stages

    torch.manual_seed(0)
    cfg = GPTConfig()
    model = GPT(cfg)
    pp = world // dp
    batch = 8
    g = torch.Generator().manual_seed(0)
    ids_all = torch.randint(0, cfg.vocab, (dp * batch, cfg.seq_len + 1), generator=g)
    ids, targets = ids_all[:, :-1].contiguous(), ids_all[:, 1:].contiguous()
    ref_loss, ref_grads, ref_params = _reference(model, ids, targets)

    n_stages = len(placement)
    stages = gpt_stages(copy.deepcopy(model), n_stages)
    names = _stage_param_names(model, n_stages)
    pp_rank, dp_rank = rank % pp, rank // pp
    mine = [s for s in range(n_stages) if placement[s] == pp_rank]
    parts = [stages[s] for s in mine]
    if split_w:
        for p in parts:
            replace_layer_with_layer_dw(p)
    pipe = Pipeline(parts, None, partitioner=False, scheduler=scheduler, placement=placement, dp=dp, outputs="device")
    my_ids = ids[dp_rank * batch : (dp_rank + 1) * batch]
    my_tgt = targets[dp_rank * batch : (dp_rank + 1) * batch]
    out, loss = pipe(my_ids, my_tgt, GPT.loss_fn, split_size=batch // nmb)
    if pipe.is_last():
        assert loss is not None
        torch.testing.assert_close(loss, ref_loss, atol=ATOL, rtol=RTOL)
        assert len(out) == nmb
    else:
        assert out is None and loss is None
    for block in pipe.blocks:
        for n, p in block.model.named_parameters():
            gname = names[(block.id, n)]
            assert p.grad is not None, gname
            torch.testing.assert_close(p.grad, ref_grads[gname], atol=ATOL, rtol=RTOL, msg=lambda m: f"{gname}: {m}")
    opt = torch.optim.AdamW(list(pipe.parameters()), lr=1e-3)
    opt.step()
    for block in pipe.blocks:
        for n, p in block.model.named_parameters():
            torch.testing.assert_close(p.detach(), ref_params[names[(block.id, n)]], atol=ATOL, rtol=RTOL)
    # a second step reuses the cached schedule and accumulates on top of zeroed grads
    pipe.zero_grad()
    pipe(my_ids, my_tgt, GPT.loss_fn, split_size=batch // nmb)
    pipe.clear()


@pytest.mark.parametrize(
    "scheduler,placement,dp,nmb,split_w",
    [
        ("1f1b", [0, 1], 1, 4, False),  # the plumbing config: pp=2, 1F1B, 4 micro-batches
        ("afab", [0, 1], 1, 4, False),
        ("zbh1", [0, 1], 1, 4, True),
        ("zbh2", [0, 1], 1, 4, True),
        ("zbv", [0, 1, 1, 0], 1, 4, True),
        ("hanayo", [0, 1, 1, 0], 1, 4, False),
        ("1f1b", [0, 1, 0, 1], 1, 4, False),
        ("full_remat", [0, 1], 1, 4, False),
    ],
)
def test_pipeline_matches_single_process(scheduler, placement, dp, nmb, split_w):
    run_ranks(_worker, len(set(placement)) * dp, scheduler, placement, dp, nmb, split_w)


@pytest.mark.parametrize("scheduler,placement", [("1f1b", [0, 1]), ("zbv", [0, 1, 1, 0]), ("zbh1", [0, 1]), ("hanayo", [0, 1, 1, 0])])
def test_data_parallel_replicas(scheduler, placement):
    run_ranks(_worker, 4, scheduler, placement, 2, 4, scheduler.startswith("zb"))


@pytest.mark.parametrize("scheduler,placement,split_w", [("zbv", [0, 1, 1, 0], True), ("1f1b", [0, 1, 0, 1], False), ("zbh1", [0, 1], True)])
def test_untagged_channels_like_nccl(scheduler, placement, split_w):
    """One communicator per channel and no tags: messages are matched by order and size only,
    as NCCL does, so a stray header or a misordered recv fails here instead of on GPUs."""
    run_ranks(_worker, 2, scheduler, placement, 1, 4, split_w, True)


def _auto_worker(rank, world, partitioner, dp):
    """Rank 0 traces, profiles and cuts the whole model; the other ranks receive their stages."""
    import copy

    from elf_b200 import Pipeline, replace_layer_with_layer_dw
    from elf_b200.models.llama import LlamaConfig, build_llama, llama_loss_fn

    torch.manual_seed(0)
    cfg = LlamaConfig(n_layers=4, d_model=64, n_heads=4, n_kv_heads=2, ffn=128, vocab=256, seq_len=32, rope_theta=10000.0)
    model = build_llama(cfg, dtype=torch.float32, seed=3)
    ref = copy.deepcopy(model)
    replace_layer_with_layer_dw(model)
    pp = world // dp
    g = torch.Generator().manual_seed(5)
    tok = torch.randint(0, cfg.vocab, (dp * 4, cfg.seq_len + 1), generator=g)
    ids, tgt = tok[:, :-1].contiguous(), tok[:, 1:].contiguous()
    pipe = Pipeline(model, ids[:1], partitioner=partitioner, scheduler="1f1b", dp=dp, outputs="device")
    assert len(pipe.signatures) == pp and len(pipe.blocks) == 1
    lo = (rank // pp) * 4
    out, loss = pipe(ids[lo : lo + 4], tgt[lo : lo + 4], llama_loss_fn, split_size=1)
    ref_loss = llama_loss_fn(ref(ids), tgt)
    ref_loss.backward()
    if pipe.is_last():
        torch.testing.assert_close(loss, ref_loss.detach(), atol=ATOL, rtol=RTOL)
    ref_grads = dict(ref.named_parameters())
    seen = 0
    for name, p in pipe.named_parameters():  # fx sub-modules keep the original qualified names
        torch.testing.assert_close(p.grad, ref_grads[name].grad, atol=ATOL, rtol=RTOL, msg=lambda m: f"{name}: {m}")
        seen += 1
    assert seen > 0
    merged = pipe.gather_parameters(dst=(rank // pp) * pp)
    if rank % pp == 0:
        assert set(merged) == set(ref_grads)
    pipe.clear()


@pytest.mark.parametrize("partitioner,world,dp", [("constrained", 2, 1), ("naive", 2, 1), ("dagP", 4, 2)])
def test_auto_partition_and_model_shipping(partitioner, world, dp):
    run_ranks(_auto_worker, world, partitioner, dp)


def _split_layer_worker(rank, world, mode=True):
    """Llama stages cut between the attention half and the MLP half of a layer, ZB-V with the
    simulator-chosen activation cap: loss and gradients equal the same stages run in sequence."""
    import functools

    from elf_b200 import Pipeline
    from elf_b200.models.llama import LlamaConfig, build_llama_stages, llama_loss_fn, llama_stage_costs, llama_stage_signatures
    from elf_b200.scheduling.schedulers import generate_zbv_schedule

    cfg = LlamaConfig(n_layers=5, d_model=64, n_heads=4, n_kv_heads=2, ffn=128, vocab=256, seq_len=32, rope_theta=10000.0)
    placement = list(range(world)) + list(range(world - 1, -1, -1))
    costs = llama_stage_costs(cfg, len(placement), placement, split_layers=mode)
    ref_stages = build_llama_stages(cfg, len(placement), dtype=torch.float32, seed=11, split_backward=False, placement=placement, split_layers=mode)
    kinds = {type(m).__name__ for s in ref_stages for m in s}
    assert {"LlamaAttentionBlock", "LlamaMLPBlock"} & kinds, kinds  # at least one layer is cut in two
    signatures = llama_stage_signatures(cfg, len(placement), placement, mode)
    if mode == "thirds":  # a boundary after the gate/up block carries the residual stream and the activation
        assert "LlamaMLPUpBlock" in kinds and "LlamaMLPDownBlock" in kinds, kinds
        assert any(sig.noutputs == 2 for sig in signatures) and any(sig.ninputs == 2 for sig in signatures)
    mine = [i for i, r in enumerate(placement) if r == rank]
    stages = build_llama_stages(cfg, len(placement), only=mine, dtype=torch.float32, seed=11, placement=placement, split_layers=mode)
    g = torch.Generator().manual_seed(5)
    tok = torch.randint(0, cfg.vocab, (6, cfg.seq_len + 1), generator=g)
    ids, tgt = tok[:, :-1].contiguous(), tok[:, 1:].contiguous()
    sched = functools.partial(generate_zbv_schedule, cap="auto", stage_costs=costs, ratios=(1.0, 1.25, 0.9))
    pipe = Pipeline([stages[i] for i in mine], None, partitioner=False, scheduler=sched, placement=placement, outputs="device", signatures=signatures)
    _, loss = pipe(ids, tgt, llama_loss_fn, split_size=1)
    x = ids
    for s in ref_stages:
        x = s(*x) if isinstance(x, tuple) else s(x)
    ref_loss = llama_loss_fn(x, tgt)
    ref_loss.backward()
    if pipe.is_last():
        torch.testing.assert_close(loss, ref_loss.detach(), atol=ATOL, rtol=RTOL)
    for block in pipe.blocks:
        ref_params = dict(ref_stages[block.id].named_parameters())
        for name, p in block.model.named_parameters():
            torch.testing.assert_close(p.grad, ref_params[name.replace(".layer.", ".")].grad if name not in ref_params else ref_params[name].grad, atol=ATOL, rtol=RTOL,
                                       msg=lambda m: f"stage {block.id} {name}: {m}")
    # profile-guided re-layout: time one step per operation, lay the schedule out again for the
    # measured (F, B, W) durations of every stage, and get the same numbers from the new schedule
    import os

    os.environ["ELF_TIMINGS"] = "1"
    try:
        pipe.zero_grad()
        pipe(ids, tgt, llama_loss_fn, split_size=1)
    finally:
        os.environ.pop("ELF_TIMINGS")
    measured = pipe.measured_stage_costs()
    assert len(measured) == len(placement) and all(len(t) == 3 and t[0] > 0 and t[1] > 0 and t[2] > 0 for t in measured)
    pipe.set_scheduler(functools.partial(generate_zbv_schedule, cap="auto", stage_costs=measured))
    pipe.zero_grad()
    _, loss2 = pipe(ids, tgt, llama_loss_fn, split_size=1)
    if pipe.is_last():
        torch.testing.assert_close(loss2, ref_loss.detach(), atol=ATOL, rtol=RTOL)
    for block in pipe.blocks:
        ref_params = dict(ref_stages[block.id].named_parameters())
        for name, p in block.model.named_parameters():
            torch.testing.assert_close(p.grad, ref_params[name.replace(".layer.", ".")].grad if name not in ref_params else ref_params[name].grad, atol=ATOL, rtol=RTOL)
    pipe.clear()


@pytest.mark.parametrize("mode", [True, "thirds"])
def test_stages_cut_inside_layers(mode):
    run_ranks(_split_layer_worker, 2, mode)


def test_thirds_cut_with_untagged_channels():
    """Two tensors per boundary over one-communicator-per-channel p2p (NCCL-like matching)."""
    import os

    os.environ["ELF_B200_P2P_STRICT"] = "1"
    try:
        run_ranks(_split_layer_worker, 2, "thirds")
    finally:
        os.environ.pop("ELF_B200_P2P_STRICT")


def _budget_worker(rank, world):
    """Llama stages (which cache rotary tables on first use) on two ranks with a memory budget: the
    shape-propagation pass of the stage profiler must leave nothing fake behind in the modules."""
    from elf_b200 import Pipeline, Placement
    from elf_b200.models.llama import LLAMA_CONFIGS, build_llama_stages, llama_loss_fn

    cfg = LLAMA_CONFIGS["llama-tiny"]
    placement = Placement.default("zbv", world)
    mine = placement.get_ids(rank)
    g = torch.Generator().manual_seed(0)
    tok = torch.randint(0, cfg.vocab, (4, cfg.seq_len + 1), generator=g)
    losses = []
    for budget in (None, 1e6):
        stages = build_llama_stages(cfg, len(placement), only=mine, device="cpu", dtype=torch.float32, seed=1, placement=list(placement))
        pipe = Pipeline([stages[i] for i in mine], tok[:1, :-1].contiguous(), partitioner=False, scheduler="zbv", placement=list(placement), outputs="none", memory_budget=budget)
        _, loss = pipe(tok[:, :-1].contiguous(), tok[:, 1:].contiguous(), llama_loss_fn, split_size=1)
        losses.append(loss)
        if budget is not None:
            assert len(pipe.get_profiling_statistics()) == len(placement)
        pipe.clear()
    if losses[0] is not None:
        torch.testing.assert_close(losses[0], losses[1], atol=1e-5, rtol=1e-5)


def test_memory_budget_on_two_ranks_with_llama_stages():
    run_ranks(_budget_worker, 2, timeout=150.0)
