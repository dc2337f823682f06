"""Failure detection and recovery, exercised on the host only: CPU tensors, gloo ranks,
fakes of the failing call.  Nothing here faults, traps or hangs a GPU.

* a rank that leaves between two steps, and a message that is never sent, surface as an
  exception on the surviving rank within the process-group timeout instead of a hang;
* an exception inside an operation (a failing loss function) leaves the pipeline usable;
* truncated, missing and wrong-stage checkpoint files give clear errors;
* the device status word written by kernels on a bounded-wait timeout turns into a Python
  exception (checked against a host-side stand-in for the status tensor);
* resuming from a checkpoint keeps the loaded weights through the next optimizer step;
* the gradient-exchange epoch advances only on steps that exchange gradients.
"""

import os
import time
from datetime import timedelta

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from elf_b200 import Pipeline, replace_layer_with_layer_dw
from elf_b200.models.gpt import GPT, GPTConfig, gpt_stages
from tests.dist_utils import _free_port

CFG = GPTConfig(n_layers=2, d_model=64, n_heads=2, ffn=128, vocab=128, seq_len=32)
PG_TIMEOUT_S = 6


def _data(batch=4, seed=1):
    g = torch.Generator().manual_seed(seed)
    tok = torch.randint(0, CFG.vocab, (batch, CFG.seq_len + 1), generator=g)
    return tok[:, :-1].contiguous(), tok[:, 1:].contiguous()


def _local_pipe(scheduler="1f1b", placement=(0, 0), dtype=None, **kw):
    torch.manual_seed(0)
    model = GPT(CFG)
    if dtype is not None:
        model = model.to(dtype)
    stages = gpt_stages(model, len(placement))
    for s in stages:
        replace_layer_with_layer_dw(s)
    return Pipeline(stages, None, partitioner=False, scheduler=scheduler, placement=list(placement), outputs="device", **kw)


# ----------------------------------------------------------------------------------------
# ranks that misbehave (gloo, CPU)
# ----------------------------------------------------------------------------------------


def _report_and_exit(results, item):
    results.put(item)
    results.close()
    results.join_thread()  # the feeder thread must have written the item before the process goes
    os._exit(0)  # skip collective teardown: the group may be broken, or this rank is "leaving"


def _two_rank_entry(rank, port, mode, results):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE="2")
    torch.set_num_threads(1)
    dist.init_process_group("gloo", rank=rank, world_size=2, timeout=timedelta(seconds=PG_TIMEOUT_S))
    torch.manual_seed(0)
    stages = gpt_stages(GPT(CFG), 2)
    for s in stages:
        replace_layer_with_layer_dw(s)
    pipe = Pipeline([stages[rank]], None, partitioner=False, scheduler="1f1b", placement=[0, 1], outputs="none")
    ids, tgt = _data()
    pipe(ids, tgt, GPT.loss_fn, split_size=1)  # a healthy step first
    dist.barrier()
    if mode == "leave" and rank == 1:
        _report_and_exit(results, (rank, "left", 0.0))  # gone between two steps, nothing of its own in flight
    if mode == "drop" and rank == 0:
        from elf_b200.execution.channels import Channel

        real_send = Channel.send

        def lossy_send(self, tensor, mb):
            if self.direction == "fwd" and mb == 2:
                return  # this message is never sent
            return real_send(self, tensor, mb)

        Channel.send = lossy_send
    t0 = time.perf_counter()
    try:
        pipe(ids, tgt, GPT.loss_fn, split_size=1)
        outcome = "no error"
    except BaseException as exc:  # noqa: BLE001 - the test wants to see whatever surfaced
        outcome = f"raised {type(exc).__name__}"
    _report_and_exit(results, (rank, outcome, time.perf_counter() - t0))


def _run_two_ranks(mode):
    ctx = mp.get_context("spawn")
    results = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_two_rank_entry, args=(r, port, mode, results), daemon=True) for r in range(2)]
    for p in procs:
        p.start()
    deadline = time.time() + 90
    for p in procs:
        p.join(max(1.0, deadline - time.time()))
    hung = [p for p in procs if p.is_alive()]
    for p in hung:
        p.terminate()
    got = {}
    while not results.empty():
        rank, what, secs = results.get()
        got[rank] = (what, secs)
    assert not hung, f"ranks hung instead of failing: {got}"
    return got


@pytest.mark.dist
def test_rank_that_leaves_between_steps_is_detected():
    got = _run_two_ranks("leave")
    assert got[1][0] == "left"
    what, secs = got[0]
    assert what.startswith("raised"), got
    assert secs < 4 * PG_TIMEOUT_S + 10, got


@pytest.mark.dist
def test_message_that_is_never_sent_times_out():
    got = _run_two_ranks("drop")
    # the receiver of the dropped activation cannot finish its step; it must fail, not hang
    what, secs = got[1]
    assert what.startswith("raised"), got
    assert secs < 4 * PG_TIMEOUT_S + 10, got


# ----------------------------------------------------------------------------------------
# an operation that raises
# ----------------------------------------------------------------------------------------


def test_exception_inside_an_operation_leaves_the_pipeline_usable():
    pipe = _local_pipe()
    ids, tgt = _data()
    calls = {"n": 0}

    def flaky_loss(out, target, **kw):
        calls["n"] += 1
        if calls["n"] == 2:
            raise ValueError("injected failure in the loss of micro-batch 1")
        return GPT.loss_fn(out, target, **kw)

    with pytest.raises(ValueError, match="injected failure"):
        pipe(ids, tgt, flaky_loss, split_size=1)
    # nothing of the broken step is left behind
    for block in pipe.blocks:
        for var in block.input_variables + [v for vs in block.output_variables for v in vs]:
            assert not var.to_process and not var.saved and not var.to_send
    pipe.zero_grad()
    _, loss = pipe(ids, tgt, GPT.loss_fn, split_size=1)
    assert torch.isfinite(loss)
    ref = _local_pipe()
    _, want = ref(ids, tgt, GPT.loss_fn, split_size=1)
    torch.testing.assert_close(loss, want)
    for p, q in zip(pipe.parameters(), ref.parameters()):
        torch.testing.assert_close(p.grad, q.grad)
    pipe.clear()


# ----------------------------------------------------------------------------------------
# checkpoints
# ----------------------------------------------------------------------------------------


def test_bad_checkpoint_files_give_clear_errors(tmp_path):
    pipe = _local_pipe()
    path = pipe.checkpoint(epoch=1, dir_path=str(tmp_path))
    with pytest.raises(FileNotFoundError, match="no checkpoint"):
        pipe.load_checkpoint(epoch=2, dir_path=str(tmp_path))
    blob = open(path, "rb").read()
    with open(path, "wb") as f:
        f.write(blob[: len(blob) // 3])  # truncated while being written
    with pytest.raises(RuntimeError, match="cannot be read"):
        pipe.load_checkpoint(epoch=1, dir_path=str(tmp_path))
    state = torch.load(pipe.checkpoint(epoch=3, dir_path=str(tmp_path)), weights_only=False)
    state["state_dict_7"] = state.pop("state_dict_1")  # a file written under another placement
    torch.save(state, path)
    with pytest.raises(RuntimeError, match=r"no entry for stage 1.*holds stages \[0, 7\]"):
        pipe.load_checkpoint(epoch=1, dir_path=str(tmp_path))
    state["state_dict_1"] = {"not_a_parameter": torch.zeros(1)}
    torch.save(state, path)
    with pytest.raises(RuntimeError, match="stage 1 does not match"):
        pipe.load_checkpoint(epoch=1, dir_path=str(tmp_path))


def test_resume_survives_the_next_optimizer_step(tmp_path):
    """bf16 parameters with fp32 master weights: after ``load_checkpoint`` a step with lr=0
    must leave the checkpointed values in place (the master copy follows the load)."""
    from elf_b200.optim import FusedAdamW

    pipe = _local_pipe(dtype=torch.bfloat16)
    opt = FusedAdamW(pipe.parameters(), lr=1e-2)
    ids, tgt = _data()
    pipe.checkpoint(epoch=0, dir_path=str(tmp_path), extra={"optimizer": opt.state_dict()})
    saved = [p.detach().clone() for p in pipe.parameters()]
    for _ in range(3):
        opt.zero_grad()
        pipe(ids, tgt, GPT.loss_fn, split_size=1)
        opt.step()
    assert any(not torch.equal(p, s) for p, s in zip(pipe.parameters(), saved))
    state = pipe.load_checkpoint(epoch=0, dir_path=str(tmp_path))
    opt.param_groups[0]["lr"] = 0.0
    opt.weight_decay = 0.0
    opt.zero_grad()
    pipe(ids, tgt, GPT.loss_fn, split_size=1)
    opt.step()
    for p, s in zip(pipe.parameters(), saved):
        assert torch.equal(p, s)
    opt.load_state_dict(state["optimizer"])  # the explicit route restores moments and step as well
    assert opt.step_count == 0


# ----------------------------------------------------------------------------------------
# device status word, seen from the host
# ----------------------------------------------------------------------------------------


class _FakeEvent:
    def __init__(self, done):
        self.done = done

    def query(self):
        return self.done


def test_kernel_status_word_becomes_an_exception(monkeypatch):
    from elf_b200.ops import gemm

    record = torch.tensor([1, 2, 30, 40], dtype=torch.int32)  # what mbar_wait leaves after its time limit
    monkeypatch.setitem(gemm._STATUS, 0, record)
    with pytest.raises(RuntimeError, match=r"kernel error 1 \(an mbarrier wait timed out\); detail=\[2, 30, 40\]"):
        gemm.check_status(0)
    assert record.tolist() == [0, 0, 0, 0]  # cleared, the next check passes
    gemm.check_status(0)

    # the non-blocking route used at step boundaries: a pinned copy plus "has the copy landed"
    host = torch.tensor([2, 5, 9, 8], dtype=torch.int32)
    monkeypatch.setitem(gemm._SNAPSHOT, 0, (host, _FakeEvent(False)))
    gemm.raise_if_failed(0)  # copy still in flight: nothing to report yet
    monkeypatch.setitem(gemm._SNAPSHOT, 0, (host, _FakeEvent(True)))
    with pytest.raises(RuntimeError, match="a wait on a peer GPU timed out"):
        gemm.raise_if_failed(0)
    gemm.raise_if_failed(0)


# ----------------------------------------------------------------------------------------
# gradient-exchange epochs
# ----------------------------------------------------------------------------------------


class _CountingSync:
    def __init__(self):
        self.begun = 0
        self.synced = 0

    def begin_step(self):
        self.begun += 1

    def __call__(self, block, batch_size):
        self.synced += 1
        block.scale_grads(batch_size)

    def close(self):
        pass


def test_exchange_epoch_only_advances_on_training_steps():
    pipe = _local_pipe()
    sync = _CountingSync()
    pipe.grad_sync = sync
    for b in pipe.blocks:
        b._grad_sync = sync
    ids, tgt = _data()
    pipe(ids, tgt, GPT.loss_fn, split_size=1)
    assert (sync.begun, sync.synced) == (1, 2)
    pipe(ids, None, None, split_size=1, scheduler="inference")
    assert (sync.begun, sync.synced) == (1, 2)  # no exchange, no new epoch
    pipe.zero_grad()
    pipe(ids, tgt, GPT.loss_fn, split_size=1)
    pipe(ids, tgt, GPT.loss_fn, split_size=1)
    assert (sync.begun, sync.synced) == (3, 6)
