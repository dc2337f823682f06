"""Split backward: LinearDW / Conv1dDW against plain autograd, stash protocol, partial replay."""

import pytest
import torch
import torch.nn as nn

from elf_b200.zb_utils import (
    Conv1dDW,
    LayerDW,
    LinearDW,
    partial_dx_recomputation,
    replace_layer_with_layer_dw,
    replace_linear_with_linear_dw,
)


def _w_pass(model, mb=0):
    for m in model.modules():
        if isinstance(m, LayerDW):
            m.move_last_computed("input", mb)
            m.move_last_computed("grad_output", mb)
            if not m.is_empty("grad_output"):
                m.backward(mb)


@pytest.mark.parametrize("bias", [True, False])
@pytest.mark.parametrize("dtype", [torch.float32, torch.complex64])
def test_linear_dw_matches_autograd(bias, dtype):
    torch.manual_seed(0)
    lin = nn.Linear(6, 5, bias=bias).to(dtype)
    ref = nn.Linear(6, 5, bias=bias).to(dtype)
    ref.load_state_dict(lin.state_dict())
    dw = LinearDW(lin)
    assert dw.weight is lin.weight
    x = torch.randn(3, 4, 6, dtype=dtype, requires_grad=True)
    xr = x.detach().clone().requires_grad_()
    g = torch.randn(3, 4, 5, dtype=dtype)
    dw(x).backward(g)
    ref(xr).backward(g)
    assert dw.weight.grad is None
    torch.testing.assert_close(x.grad, xr.grad)
    _w_pass(dw)
    torch.testing.assert_close(dw.weight.grad, ref.weight.grad)
    if bias:
        torch.testing.assert_close(dw.bias.grad, ref.bias.grad)
    assert dw.is_empty("input") and dw.is_empty("grad_output")
    # a second micro-batch accumulates
    dw(x).backward(g)
    _w_pass(dw, 1)
    torch.testing.assert_close(dw.weight.grad, 2 * ref.weight.grad)


@pytest.mark.parametrize("kwargs", [dict(), dict(stride=2, padding=1), dict(padding="same", dilation=2), dict(groups=2)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.complex64])
def test_conv1d_dw_matches_autograd(kwargs, dtype):
    torch.manual_seed(1)
    conv = nn.Conv1d(4, 6, 3, **kwargs).to(dtype)
    ref = nn.Conv1d(4, 6, 3, **kwargs).to(dtype)
    ref.load_state_dict(conv.state_dict())
    dw = Conv1dDW(conv)
    x = torch.randn(2, 4, 11, dtype=dtype, requires_grad=True)
    xr = x.detach().clone().requires_grad_()
    y, yr = dw(x), ref(xr)
    g = torch.randn_like(y)
    y.backward(g)
    yr.backward(g)
    torch.testing.assert_close(y, yr)
    torch.testing.assert_close(x.grad, xr.grad, atol=1e-5, rtol=1e-5)
    _w_pass(dw)
    torch.testing.assert_close(dw.weight.grad, ref.weight.grad, atol=1e-4, rtol=1e-4)
    torch.testing.assert_close(dw.bias.grad, ref.bias.grad, atol=1e-5, rtol=1e-5)


def test_replace_helpers_and_stash_api():
    model = nn.Sequential(nn.Linear(4, 4), nn.ReLU(), nn.Conv1d(2, 2, 1), nn.Linear(4, 4))
    replace_layer_with_layer_dw(model, only=[nn.Linear])
    assert isinstance(model[0], LinearDW) and isinstance(model[3], LinearDW) and not isinstance(model[2], LayerDW)
    replace_layer_with_layer_dw(model)
    assert isinstance(model[2], Conv1dDW)
    m2 = nn.Sequential(nn.Linear(4, 4))
    replace_linear_with_linear_dw(m2, "cpu")
    assert isinstance(m2[0], LinearDW)
    layer = m2[0]
    layer.set("input", 2, torch.ones(1))
    assert layer._state() == "(1,0)" and not layer.is_empty("input")
    with pytest.raises(ValueError):
        layer.set("input", 2, torch.ones(1))
    layer.delete("input", 2)
    with pytest.raises(ValueError):
        layer.delete("input", 2)
    with pytest.raises(ValueError):
        layer.backward(0)
    layer.clear()
    assert layer.ctx == {"input": [], "grad_output": []}


def test_module_reuse_sums_output_grads():
    torch.manual_seed(0)
    lin = LinearDW(nn.Linear(4, 4))
    ref = nn.Linear(4, 4)
    ref.load_state_dict(lin.state_dict())
    x = torch.randn(2, 4)
    # same input twice so that one stashed input serves both uses
    (lin(x) + lin(x)).sum().backward()
    (ref(x) + ref(x)).sum().backward()
    _w_pass(lin)
    torch.testing.assert_close(lin.weight.grad, ref.weight.grad)


def test_partial_dx_recomputation_refills_grad_stash_only():
    torch.manual_seed(0)
    model = replace_layer_with_layer_dw(nn.Sequential(nn.Linear(4, 4), nn.LayerNorm(4), nn.Linear(4, 3)))
    x = torch.randn(5, 4, requires_grad=True)
    y = model(x)
    g = torch.randn_like(y)
    y.backward(g, retain_graph=True)
    want = [m.last_grad_output.clone() for m in model if isinstance(m, LayerDW)]
    ln_grad = model[1].weight.grad.clone()
    for m in model:
        if isinstance(m, LayerDW):
            m.last_grad_output = None
    partial_dx_recomputation(y, g)
    got = [m.last_grad_output for m in model if isinstance(m, LayerDW)]
    for a, b in zip(got, want):
        torch.testing.assert_close(a, b)
    torch.testing.assert_close(model[1].weight.grad, ln_grad)  # non-split parameters were not touched again
