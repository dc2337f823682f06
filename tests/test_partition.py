"""Graph front-end: tracers, node profiler, every registered partitioner, stage modules."""

import pytest
import torch
import torch.nn as nn

from elf_b200.partitioners import PartitionResult, partition, profile_operations, split, trace
from elf_b200.partitioners.custom import cut_widths
from elf_b200.partitioners.utils import partition_to_dot, prune_graph, remove_inplace_leaves
from elf_b200.registry import PARTITIONERS, TRACERS
from elf_b200.zb_utils import LinearDW, replace_layer_with_layer_dw


class MLP(nn.Module):
    def __init__(self, n=24, d=32):
        super().__init__()
        self.layers = nn.ModuleList([nn.Linear(d, d) for _ in range(n)])

    def forward(self, x):
        for l in self.layers:
            x = torch.relu(l(x))
        return x


class TwoInputs(nn.Module):
    def __init__(self, d=16):
        super().__init__()
        self.a, self.b = nn.Linear(d, d), nn.Linear(d, d)
        self.tail = nn.Sequential(*[nn.Linear(d, d) for _ in range(6)])

    def forward(self, x, y):
        return self.tail(self.a(x) + self.b(y))


class SkipTwoOutputs(nn.Module):
    def __init__(self, d=16):
        super().__init__()
        self.f = nn.Sequential(*[nn.Linear(d, d) for _ in range(4)])
        self.g = nn.Sequential(*[nn.Linear(d, d) for _ in range(4)])

    def forward(self, x):
        h = self.f(x)
        return self.g(h) + x, h.sum(-1)


def run_chain(result: PartitionResult, inputs: dict):
    env = dict(inputs)
    for part, sig in zip(result.create_blocks(), result.signatures):
        outs = part(*[env[name] for name in sig.inputs])
        assert isinstance(outs, tuple) and len(outs) == len(sig.outputs)
        env.update(zip(sig.outputs, outs))
    return env


@pytest.mark.parametrize("partitioner", ["naive", "constrained", "metis", "dagP"])
@pytest.mark.parametrize("n", [1, 2, 3, 4])
def test_mlp_partitions_reproduce_the_model(partitioner, n):
    torch.manual_seed(0)
    model = MLP()
    x = torch.randn(4, 32)
    expected = model(x)
    res = partition(model, n, x, partitioner=partitioner, tracer="fx")
    assert res.n == n and len(res.signatures) == n
    res.validate()
    for blk, sig in zip(res.create_blocks(), res.signatures):
        assert isinstance(blk, torch.fx.GraphModule)
        assert sum(nd.op == "placeholder" for nd in blk.graph.nodes) == sig.ninputs
    env = run_chain(res, {"x": x})
    final = [o for sig in res.signatures for o, t in zip(sig.outputs, sig.targets) if t == [None]]
    assert len(final) == 1
    torch.testing.assert_close(env[final[0]], expected)
    n_nodes = sum(len(p) for p in res.parts)
    assert n_nodes == sum(nd.op not in ("placeholder", "output") for nd in res.graph_module.graph.nodes)
    assert res.balance_score >= 1.0 and res.transfer_score >= 0.0
    assert "PartitionResult" in repr(res)


@pytest.mark.parametrize("partitioner", ["naive", "constrained", "metis", "dagP"])
def test_two_inputs_and_two_outputs(partitioner):
    torch.manual_seed(1)
    m = TwoInputs()
    x, y = torch.randn(3, 16), torch.randn(3, 16)
    res = partition(m, 3, (x, y), partitioner=partitioner, tracer="fx")
    env = run_chain(res, {"x": x, "y": y})
    final = [o for sig in res.signatures for o, t in zip(sig.outputs, sig.targets) if None in t]
    torch.testing.assert_close(env[final[0]], m(x, y))

    m2 = SkipTwoOutputs()
    res2 = partition(m2, 2, x, partitioner=partitioner, tracer="fx")
    env2 = run_chain(res2, {"x": x})
    outs = [env2[o] for sig in res2.signatures for o, t in zip(sig.outputs, sig.targets) if None in t]
    exp = m2(x)
    assert len(outs) == 2
    for got in outs:
        assert any(got.shape == e.shape and torch.allclose(got, e, atol=1e-6) for e in exp)
    # the skip connection makes the model input an input of the second part too
    for sig in res2.signatures[1:]:
        for name, src in zip(sig.inputs, sig.sources):
            assert src is None or src < res2.signatures.index(sig)


def test_constrained_prefers_single_tensor_cuts():
    torch.manual_seed(0)
    res = partition(MLP(), 4, torch.randn(4, 32), partitioner="constrained", tracer="fx")
    assert all(sig.ninputs == 1 and sig.noutputs == 1 for sig in res.signatures)
    assert res.balance_score < 1.6


def test_layer_dw_is_a_leaf_for_every_tracer():
    model = replace_layer_with_layer_dw(MLP(4))
    x = torch.randn(2, 32)
    for key in ("fx", "fx_safe", "default"):
        gm = trace(model, x, key)
        mods = [nd for nd in gm.graph.nodes if nd.op == "call_module"]
        assert len(mods) == 4 and all(isinstance(gm.get_submodule(nd.target), LinearDW) for nd in mods)


def test_fx_safe_turns_untraceable_modules_into_leaves():
    class DataDependent(nn.Module):
        def forward(self, x):
            return x * 2 if x.sum() > 0 else x  # python control flow on a tensor value

    model = nn.Sequential(nn.Linear(8, 8), DataDependent(), nn.Linear(8, 8))
    with pytest.raises(Exception):
        TRACERS["fx"](model, None)
    gm = TRACERS["fx_safe"](model, torch.randn(2, 8))
    assert any(nd.op == "call_module" and isinstance(gm.get_submodule(nd.target), DataDependent) for nd in gm.graph.nodes)
    gm2 = TRACERS["default"](model, torch.randn(2, 8))
    x = torch.ones(2, 8)
    torch.testing.assert_close(gm2(x), model(x))


def test_export_tracer_keeps_weights_with_their_users():
    torch.manual_seed(0)
    model = MLP(6, 16)
    x = torch.randn(2, 16)
    res = partition(model, 3, x, partitioner="constrained", tracer="export")
    for sig in res.signatures[1:]:
        assert all("weight" not in name and "bias" not in name for name in sig.inputs), sig
    env = run_chain(res, {res.signatures[0].inputs[0]: x})
    final = [o for sig in res.signatures for o, t in zip(sig.outputs, sig.targets) if None in t]
    torch.testing.assert_close(env[final[0]], model(x))


def test_remove_inplace_leaves_keeps_values_and_grads():
    class M(nn.Module):
        def __init__(self):
            super().__init__()
            self.lin = nn.Linear(8, 8)
            self.act = nn.ReLU(inplace=True)

        def forward(self, x):
            y = torch.relu_(x.view(-1, 8))  # in place on a view of the stage input
            return self.act(self.lin(y))

    m = M()
    gm = torch.fx.symbolic_trace(m)
    remove_inplace_leaves(gm)
    x = torch.randn(4, 8, requires_grad=True)
    out = gm(x)  # would raise "a leaf Variable that requires grad is being used in an in-place operation"
    out.sum().backward()
    ref_x = x.detach().clone().requires_grad_()
    ref = torch.relu(m.lin(torch.relu(ref_x)))

    class Direct(nn.Module):
        def __init__(self):
            super().__init__()
            self.act = nn.ReLU(inplace=True)

        def forward(self, x):
            return self.act(x) * 2

    gm2 = torch.fx.symbolic_trace(Direct())
    remove_inplace_leaves(gm2)
    leaf = torch.randn(3, requires_grad=True)
    gm2(leaf).sum().backward()
    assert leaf.grad is not None
    ref.sum().backward()
    torch.testing.assert_close(out, ref)
    torch.testing.assert_close(x.grad, ref_x.grad)


def test_prune_and_profile_and_dot():
    class Dead(nn.Module):
        def forward(self, x):
            _unused = x * 3
            return x + 1

    gm = torch.fx.symbolic_trace(Dead())
    n_before = len(gm.graph.nodes)
    prune_graph(gm)
    assert len(gm.graph.nodes) == n_before - 1
    model = MLP(3, 8)
    gm = TRACERS["fx"](model, None)
    times, mems = profile_operations(gm, torch.randn(2, 8), niter=2)
    for nd in gm.graph.nodes:
        assert nd.name in times and nd.name in mems
    assert mems["x"] == 2 * 8 * 4
    width, ok = cut_widths(list(gm.graph.nodes), mems)
    assert max(width) >= 1 and all(ok)
    res = split(gm, times, mems, 2, "naive")
    dot = partition_to_dot(res.parts)
    assert dot.startswith("digraph") and "cluster_1" in dot


def test_custom_partitioner_via_registry():
    def halves(graph, times, memories, n):
        nodes = list(graph.graph.nodes)
        k = len(nodes) // n
        return [nodes[i * k : (i + 1) * k if i < n - 1 else None] for i in range(n)]

    PARTITIONERS.register("test_halves", halves, "equal node counts")
    try:
        res = partition(MLP(6, 8), 2, torch.randn(2, 8), partitioner="test_halves", tracer="fx")
        assert res.n == 2
    finally:
        PARTITIONERS.unregister("test_halves")


def test_native_min_volume_solver_matches_python():
    """The C++ cut solver of the host runtime returns the same cuts as the Python reference
    implementation on random instances (and the same "no solution" verdicts)."""
    import random

    from elf_b200.partitioners import dag

    if dag._native_solver() is None:
        pytest.skip("native extension not built")
    rng = random.Random(0)
    for trial in range(60):
        n = rng.randint(6, 80)
        parts = rng.randint(2, min(8, n // 2))
        times = [rng.choice([0.0, 0.5, 1.0, 2.0, 5.0]) for _ in range(n)]
        prefix = [0.0]
        for t in times:
            prefix.append(prefix[-1] + t)
        cost = [rng.choice([1.0, 2.0, 8.0, 64.0]) for _ in range(n + 1)]
        allowed = [rng.random() < 0.8 for _ in range(n + 1)]
        cap = rng.choice([1.05, 1.3, 2.0]) * prefix[-1] / parts
        got = dag._solve(prefix, cost, allowed, parts, cap, native=True)
        want = dag._solve(prefix, cost, allowed, parts, cap, native=False)
        if want is None or len(want) != parts - 1:
            assert got is None or len(got) != parts - 1
            continue
        assert got is not None
        vol = lambda cuts: sum(cost[c] for c in cuts)
        assert abs(vol(got) - vol(want)) < 1e-9  # equal optimum (ties may pick different cuts)
        bounds = [0] + got + [n]
        assert all(prefix[b] - prefix[a] <= cap + 1e-9 for a, b in zip(bounds, bounds[1:]))
        assert all(allowed[c] for c in got)
