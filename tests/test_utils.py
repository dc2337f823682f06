import pytest
import torch
import torch.nn as nn

from elf_b200.utils import TensorMetadata, Timer, TimerCPU, pretty_print_params, prod
from elf_b200.utils.flops import attention_flops, linear_flops, transformer_step_flops
from tests.dist_utils import run_ranks


def test_tensor_metadata_roundtrip():
    for dtype in (torch.float32, torch.bfloat16, torch.int64, torch.bool):
        meta = TensorMetadata(torch.empty(3, 5, 7, dtype=dtype))
        back = TensorMetadata.from_tensor(meta.to_tensor("cpu"), device="cpu")
        assert back == meta and back.shape == [3, 5, 7] and back.dtype == dtype
    big = TensorMetadata(shape=[1 << 30, 3], dtype=torch.float16)
    assert TensorMetadata.from_tensor(big.to_tensor("cpu")).shape == [1 << 30, 3]  # exact beyond 2**24
    scalar = TensorMetadata(shape=[], dtype=torch.float32, device="cpu")
    assert TensorMetadata.from_tensor(scalar.to_tensor("cpu")).shape == []
    buf = TensorMetadata(shape=[4, 2], dtype=torch.float32, device="cpu").get_buffer(3)
    assert buf.shape == (3, 4, 2) and TensorMetadata(shape=[4, 2], dtype=torch.float32).nbytes(3) == 96
    with pytest.raises(ValueError):
        TensorMetadata(shape=[1] * 15, dtype=torch.float32).to_tensor("cpu")


def test_timers_and_misc():
    with Timer("cpu", "x") as t:
        sum(range(1000))
    assert isinstance(t, TimerCPU) and t.name == "x" and t.time() >= 0
    assert isinstance(Timer(type_="cpu"), TimerCPU)
    assert pretty_print_params(8.03e9) == "8.0B" and pretty_print_params(1.5e6) == "1.5M" and pretty_print_params(12) == "12"
    assert prod([2, 3, 4]) == 24 and prod(5) == 5
    assert linear_flops(2, 3, 4) == 48
    assert attention_flops(1, 2, 8, 4, causal=False) == 2 * 2 * 2 * 8 * 8 * 4
    assert transformer_step_flops(2, 64, 4, 2, 128, 256, 32, 64) > 0


def test_flop_formulas_registered():
    from torch.utils.flop_counter import FlopCounterMode

    x = torch.randn(8, 8)
    with FlopCounterMode(display=False) as fc:
        torch.nn.functional.gelu(x) + x
    assert fc.get_total_flops() == 34 * 64 + 64


def _ship(rank, world):
    import torch.distributed as dist

    from elf_b200.utils import broadcast_models, recv_models, send_models

    torch.manual_seed(0)
    shared = nn.Linear(4, 4)
    model = nn.Sequential(nn.Linear(4, 4), nn.BatchNorm1d(4), shared, shared).double()
    model[0] = model[0].float()
    if rank == 0:
        send_models([model, nn.ReLU()], dst=1)
        got = None
    else:
        box = [None, None]
        recv_models(box, src=0)
        got = box[0]
        assert isinstance(box[1], nn.ReLU)
        for (n1, p1), (n2, p2) in zip(model.named_parameters(), got.named_parameters()):
            assert n1 == n2 and p1.dtype == p2.dtype and torch.equal(p1, p2) and p2.requires_grad == p1.requires_grad
        for (n1, b1), (n2, b2) in zip(model.named_buffers(), got.named_buffers()):
            assert n1 == n2 and torch.equal(b1, b2)
        assert got[2].weight is got[3].weight or torch.equal(got[2].weight, got[3].weight)
    box = [model if rank == 0 else None]
    broadcast_models(box, src=0)
    for p1, p2 in zip(model.parameters(), box[0].parameters()):
        assert torch.equal(p1, p2)
    dist.barrier()


@pytest.mark.dist
def test_model_shipping_between_ranks():
    run_ranks(_ship, 2)
