"""Peer-memory gradient exchange: fused weight-gradient GEMM + push, copy push, finalize.

One GPU hosts two (or four) *virtual replicas* whose "peer" buffers are ordinary buffers of
the same device; the kernels of the replicas run back to back on one stream (none of them
waits for a later launch).  The result is compared with the average of the replicas' fp32
reference gradients."""

import pytest
import torch

pytestmark = pytest.mark.gpu


def _replica(seed, dims, dev):
    torch.manual_seed(seed)
    layers = torch.nn.Sequential(*[torch.nn.Linear(i, o, bias=False) for i, o in dims], torch.nn.LayerNorm(dims[-1][1])).to(dev).to(torch.bfloat16)
    return layers


@pytest.mark.parametrize("world", [2, 4])
def test_fused_dw_push_and_finalize(world):
    from elf_b200.ops import gemm as G
    from elf_b200.parallel.dp_sync import _build_exchange
    from elf_b200.parallel.symm import LocalSymmetricGroup
    from elf_b200.zb_utils import LinearDW, replace_layer_with_layer_dw

    dev = torch.device("cuda", 0)
    dims = [(256, 512), (512, 264), (264, 128)]
    group = LocalSymmetricGroup(world, dev)
    reps, exchanges = [], []
    base = _replica(0, dims, dev)
    for r in range(world):
        m = _replica(0, dims, dev)
        m.load_state_dict(base.state_dict())
        replace_layer_with_layer_dw(m)
        layers = [l for l in m.modules() if isinstance(l, LinearDW)]
        ex = _build_exchange(list(m.parameters()), layers, group.allocator(r), r, world, timeout_ms=500.0)
        reps.append(m)
        exchanges.append(ex)
    n_mb, batch = 3, 4
    for step in range(2):  # two steps: both inbox parities, growing epochs
        ref_grads = None
        for r, (m, ex) in enumerate(zip(reps, exchanges)):
            ex.flat.zero_grad()
            ex.begin_step()
            ref = _replica(0, dims, dev).float()
            ref.load_state_dict({k: v.float() for k, v in base.state_dict().items()})
            for mb in range(n_mb):
                torch.manual_seed(100 * step + 10 * r + mb)
                x = torch.randn(batch, 64, dims[0][0], device=dev, dtype=torch.bfloat16)
                y = m(x)
                g = torch.randn_like(y)
                y.backward(g)
                for l in m.modules():
                    if isinstance(l, LinearDW):
                        l.move_last_computed("input", mb)
                        l.move_last_computed("grad_output", mb)
                        l._final_pass = mb == n_mb - 1
                        l.backward(mb)
                ref(x.float()).backward(g.float())
            grads = [p.grad.clone() for p in ref.parameters()]
            ref_grads = grads if ref_grads is None else [a + b for a, b in zip(ref_grads, grads)]
        scale = 1.0 / (n_mb * batch * world)
        for ex in exchanges:  # all pushes first: on one GPU a finalize must not wait for a later launch
            ex.push_rest()
        for ex in exchanges:
            ex.reduce(scale)
        torch.cuda.synchronize()
        G.check_status()
        for m in reps:
            for p, want in zip(m.parameters(), ref_grads):
                err = ((p.grad.float() - want * scale).norm() / (want * scale).norm()).item()
                assert err < 2e-2, err
        assert all(len(ex.pushed) == 3 for ex in exchanges)  # the three matrices went out through GEMM epilogues


def test_finalize_wait_is_bounded():
    """A flag that nobody raises: the wait gives up after its limit, reports it in the
    status word, and the context stays usable."""
    from elf_b200.ops import _ext, gemm as G

    dev = torch.device("cuda", 0)
    grad = torch.ones(1024, device=dev, dtype=torch.bfloat16)
    inbox = torch.ones(1024, device=dev, dtype=torch.bfloat16)
    flags = torch.zeros(4, device=dev, dtype=torch.int32)
    wait = torch.tensor([0], device=dev, dtype=torch.int32)
    status = G.status(dev)
    status.zero_()
    _ext.get().finalize_reduce(grad, inbox, 1, flags, 1, wait, 5, 0.5, 100.0, status)
    torch.cuda.synchronize()
    rec = status.tolist()
    assert rec[0] == 2 and rec[2] == 5 and rec[3] == 0  # peer timeout, waited-for epoch, value seen
    with pytest.raises(RuntimeError, match="peer GPU timed out"):
        G.check_status(dev)
    assert torch.allclose(grad.float(), torch.ones(1024, device=dev))  # (1 + 1) * 0.5: the reduction still ran
    y = torch.ones(8, device=dev) * 2  # the context still works
    assert y.sum().item() == 16
