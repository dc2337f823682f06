"""Pure (no torch.distributed, no GPU) checks of the schedule zoo, comm insertion and the
three comm schedulers, with the timeline simulator and the protocol replay as oracles."""

from collections import Counter

import pytest

from elf_b200 import Placement, sequential_signatures
from elf_b200.partitioners.signature import Signature
from elf_b200.registry import COMM_SCHEDULERS, SCHEDULERS
from elf_b200.scheduling import (
    DeadlockError,
    Operation,
    OperationType,
    OpOptions,
    add_comms,
    check_schedule_validity,
    replay_comms,
    schedule_to_str,
    simulate,
)
from elf_b200.scheduling.schedulers import FixedSchedule

T = OperationType


def compute_trace(schedule, rank):
    letters = {T.FORWARD: "f", T.BACKWARD_INPUTS: "b", T.BACKWARD_PARAMS: "w"}
    return [f"{letters[op.op]}{op.block_id}-{op.mb_id}" for op in schedule if op.rank == rank and op.op in letters]


def test_afab_exact_sequence():
    sched = SCHEDULERS["afab"]([0, 1], 2)
    assert compute_trace(sched, 0) == ["f0-0", "f0-1", "b0-0", "w0-0", "b0-1", "w0-1"]
    assert compute_trace(sched, 1) == ["f1-0", "f1-1", "b1-0", "w1-0", "b1-1", "w1-1"]
    loss = [op.op for op in sched if op.rank == 1 and op.op in (T.LOSS_FORWARD, T.LOSS_BACKWARD)]
    assert loss == [T.LOSS_FORWARD, T.LOSS_FORWARD, T.LOSS_BACKWARD, T.LOSS_BACKWARD]
    assert SCHEDULERS["gpipe"] is SCHEDULERS["afab"]


def test_1f1b_exact_sequence():
    sched = SCHEDULERS["1f1b"]([0, 1], 4)
    assert compute_trace(sched, 0) == ["f0-0", "f0-1", "b0-0", "w0-0", "f0-2", "b0-1", "w0-1", "f0-3", "b0-2", "w0-2", "b0-3", "w0-3"]
    assert compute_trace(sched, 1) == ["f1-0", "b1-0", "w1-0", "f1-1", "b1-1", "w1-1", "f1-2", "b1-2", "w1-2", "f1-3", "b1-3", "w1-3"]


def test_zbh1_defers_w():
    sched = SCHEDULERS["zbh1"]([0, 1, 2, 3], 8)
    assert compute_trace(sched, 0)[:9] == ["f0-0", "f0-1", "f0-2", "f0-3", "b0-0", "w0-0", "f0-4", "b0-1", "w0-1"]
    tr3 = compute_trace(sched, 3)
    assert tr3[:8] == ["f3-0", "b3-0", "f3-1", "b3-1", "f3-2", "b3-2", "f3-3", "b3-3"]  # lag = depth 3
    assert tr3[8] == "w3-0"


CASES = [
    ("afab", [0, 1]),
    ("afab", [0, 1, 2, 3]),
    ("afab", [0, 0, 1, 1]),
    ("1f1b", [0, 1]),
    ("1f1b", [0, 1, 2, 3]),
    ("1f1b", [0, 1, 0, 1]),
    ("megatron", [0, 1, 2, 3, 0, 1, 2, 3]),
    ("1f1b", [0, 1, 2, 0, 1, 2, 0, 1, 2]),
    ("hanayo", [0, 1, 1, 0]),
    ("hanayo", [0, 1, 2, 3, 3, 2, 1, 0]),
    ("hanayo", [0, 1, 1, 0, 0, 1, 1, 0]),
    ("hanayo", list(Placement.v_shape(8))),
    ("zbh1", [0, 1]),
    ("zbh1", [0, 1, 2, 3]),
    ("zbh2", [0, 1]),
    ("zbh2", [0, 1, 2, 3]),
    ("zbv", [0, 1, 1, 0]),
    ("zbv", list(Placement.v_shape(4))),
    ("zbv", list(Placement.v_shape(8))),
    ("zbv", [0, 0]),
    ("full_remat", [0, 1, 2, 3]),
]


@pytest.mark.parametrize("name,placement", CASES)
@pytest.mark.parametrize("nmb", [2, 4, 8, 13])
@pytest.mark.parametrize("comm", ["topo", "simulation", "pipelined"])
def test_structure_and_protocol(name, placement, nmb, comm):
    n_stages = len(placement)
    sched = SCHEDULERS[name](placement, nmb)
    sched = add_comms(sched, sequential_signatures(placement))
    sched = COMM_SCHEDULERS[comm](sched)
    check_schedule_validity(sched)
    counts = Counter(op.op for op in sched)
    for kind in (T.FORWARD, T.BACKWARD_INPUTS, T.BACKWARD_PARAMS, T.RECV_FORWARD, T.SEND_FORWARD, T.RECV_BACKWARD, T.SEND_BACKWARD):
        assert counts[kind] == n_stages * nmb, (kind, counts[kind])
    assert counts[T.LOSS_FORWARD] == counts[T.LOSS_BACKWARD] == nmb
    assert counts[T.ALL_REDUCE_PARAM_GRADS] == n_stages
    for rank in set(placement):
        prog = [op for op in sched if op.rank == rank]
        pos = {}
        for i, op in enumerate(prog):
            pos.setdefault((op.op, op.block_id, op.mb_id), i)
        for (kind, s, mb), i in pos.items():
            if kind is T.BACKWARD_INPUTS:
                assert pos[(T.FORWARD, s, mb)] < i <= pos[(T.BACKWARD_PARAMS, s, mb)]
                if s == n_stages - 1:
                    assert pos[(T.FORWARD, s, mb)] < pos[(T.LOSS_FORWARD, s, mb)] < pos[(T.LOSS_BACKWARD, s, mb)] < i
            if kind is T.ALL_REDUCE_PARAM_GRADS:
                assert all(j < i for (k2, s2, _), j in pos.items() if k2 is T.BACKWARD_PARAMS and s2 == s)
            if kind is T.FORWARD:
                assert all(pos[(T.RECV_FORWARD, s, mb)] < i for _ in [0])
                assert pos[(T.SEND_FORWARD, s, mb)] > i
    replay_comms(sched, placement)  # raises DeadlockError on a protocol violation
    sim = simulate(sched, placement)
    assert sim.makespan >= 3 * nmb * n_stages / len(set(placement))


@pytest.mark.parametrize("name,pp", [("1f1b", 4), ("zbv", 4), ("hanayo", 4), ("zbh1", 4), ("zbh2", 4)])
def test_data_parallel_offset_does_not_change_the_program(name, pp):
    """Schedulers see pipeline-local placements, but must also cope with shifted ones:
    the program of replica 1 is the program of replica 0 with ranks shifted."""
    base = Placement.default(name, pp)
    a = SCHEDULERS[name](base, 8)
    b = SCHEDULERS[name](base.add_offset(pp), 8)
    assert len(a) == len(b) > 0
    assert [(o.op, o.block_id, o.mb_id, o.rank + pp) for o in a] == [(o.op, o.block_id, o.mb_id, o.rank) for o in b]


@pytest.mark.parametrize("pp,nmb", [(2, 4), (4, 8), (4, 12), (8, 16), (8, 32), (4, 7)])
def test_zbv_any_number_of_micro_batches(pp, nmb):
    placement = Placement.default("zbv", pp)
    sim = simulate(SCHEDULERS["zbv"](placement, nmb), placement)
    assert max(sim.peak_live.values()) <= 2 * pp  # the footprint of 1F1B
    ideal = 3 * 2 * nmb
    assert sim.makespan <= ideal + 3 * pp  # close to bubble-free
    one_f_one_b = simulate(SCHEDULERS["1f1b"](list(range(pp)), nmb), list(range(pp)))
    assert sim.makespan / 2 <= one_f_one_b.makespan  # per-stage work is half: compare like with like


def test_zero_bubble_beats_1f1b():
    pl = [0, 1, 2, 3]
    m = {n: simulate(SCHEDULERS[n](pl, 8), pl).makespan for n in ("afab", "1f1b", "zbh1", "zbh2")}
    assert m["zbh1"] < m["1f1b"] <= m["afab"]
    assert m["zbh2"] <= m["zbh1"]


def test_inference_has_no_backward():
    sched = add_comms(SCHEDULERS["inference"]([0, 1, 2], 4), sequential_signatures([0, 1, 2]))
    kinds = {op.op for op in sched}
    assert T.BACKWARD_INPUTS not in kinds and T.LOSS_FORWARD not in kinds and T.RECV_BACKWARD not in kinds
    assert sum(op.op is T.FORWARD for op in sched) == 12
    replay_comms(COMM_SCHEDULERS["pipelined"](sched), [0, 1, 2])


def test_fixed_schedule_replays_order():
    order = [("f", 0, 0), ("f", 1, 0), ("b", 1, 0), ("w", 1, 0), ("b", 0, 0), ("w", 0, 0)]
    sched = FixedSchedule({"order": order})([0, 1], 1)
    assert compute_trace(sched, 0) == ["f0-0", "b0-0", "w0-0"]
    assert compute_trace(sched, 1) == ["f1-0", "b1-0", "w1-0"]
    assert SCHEDULERS["fixed"] is FixedSchedule


def test_full_remat_marks_forwards():
    sched = SCHEDULERS["full_remat"]([0, 1], 2)
    f0 = [op for op in sched if op.rank == 0 and op.op is T.FORWARD]
    f1 = [op for op in sched if op.rank == 1 and op.op is T.FORWARD]
    assert all(op.options[OpOptions.REMAT_STRATEGY]("", None) for op in f0)
    assert all(OpOptions.REMAT_STRATEGY not in op.options for op in f1)
    assert "F0-0" in schedule_to_str(sched)


def test_add_comms_with_skip_connection():
    # stage 0 feeds stages 1 and 2; stage 2 takes inputs from 0 and 1
    sigs = [
        Signature(["x"], ["a"], [None], [[1, 2]]),
        Signature(["a"], ["b"], [0], [[2]]),
        Signature(["a", "b"], ["out"], [0, 1], [[None]]),
    ]
    placement = [0, 1, 2]
    sched = add_comms(SCHEDULERS["afab"](placement, 2), sigs)
    sends0 = [op.options["dst"] for op in sched if op.block_id == 0 and op.mb_id == 0 and op.op is T.SEND_FORWARD]
    assert sends0 == [1, 2]
    recvs2 = [op.options["src"] for op in sched if op.block_id == 2 and op.mb_id == 0 and op.op is T.RECV_FORWARD]
    assert recvs2 == [1, 0]  # sources in descending order
    rb0 = [op.options["src"] for op in sched if op.block_id == 0 and op.mb_id == 0 and op.op is T.RECV_BACKWARD]
    assert rb0 == [1, 2]
    for comm in ("topo", "simulation", "pipelined"):
        replay_comms(COMM_SCHEDULERS[comm](list(sched)), placement)


def test_replay_detects_a_deadlock():
    placement = [0, 1]
    sched = add_comms(SCHEDULERS["afab"](placement, 1), sequential_signatures(placement))
    good = COMM_SCHEDULERS["topo"](sched)
    # rank 1 computes its forward before posting the recv it depends on
    bad = [op for op in good if not (op.op is T.RECV_FORWARD and op.block_id == 1)]
    bad += [op for op in good if op.op is T.RECV_FORWARD and op.block_id == 1]
    with pytest.raises(DeadlockError):
        replay_comms(bad, placement)


def test_operation_equality_and_hash_agree():
    a = Operation(0, 1, T.FORWARD, 0)
    b = Operation(1, 1, T.FORWARD, 0)
    assert a != b and a == Operation(0, 1, T.FORWARD, 0)
    assert hash(a) == hash(Operation(0, 1, T.FORWARD, 0))


def test_schedule_compile_is_fast():
    import time

    placement = Placement.default("zbv", 8)
    t0 = time.perf_counter()
    s = add_comms(SCHEDULERS["zbv"](placement, 32), sequential_signatures(placement))
    s = COMM_SCHEDULERS["pipelined"](s)
    assert len(s) == 3664
    assert time.perf_counter() - t0 < 2.0


@pytest.mark.parametrize("pp", [2, 4, 8])
def test_headline_zbv_configuration_replays_without_deadlock(pp):
    """The schedule the benchmark runs (V placement, 16 micro-batches, stages cut inside layers for
    the 8B shape, simulator-chosen activation cap) is valid and its p2p protocol replays on every
    comm scheduler."""
    from elf_b200.models.llama import LLAMA_CONFIGS, llama_stage_costs
    from elf_b200.scheduling.schedulers import generate_zbv_schedule

    placement = list(range(pp)) + list(range(pp - 1, -1, -1))
    costs = llama_stage_costs(LLAMA_CONFIGS["llama3-8b"], 2 * pp, placement, split_layers=True)
    sched = generate_zbv_schedule(placement, 16, cap="auto", cap_limit=6 * pp, stage_costs=costs, ratios=(1.0, 1.25, 0.9))
    assert sum(op.op is T.FORWARD for op in sched) == 2 * pp * 16
    assert sum(op.op is T.BACKWARD_PARAMS for op in sched) == 2 * pp * 16
    full = add_comms(sched, sequential_signatures(placement))
    for comm in ("topo", "pipelined"):
        ordered = COMM_SCHEDULERS[comm](list(full))
        check_schedule_validity(ordered)
        replay_comms(ordered, placement)


def test_robust_zbv_layout_is_valid_and_deterministic():
    """``robust > 0``: candidates laid out for perturbed costs, scored over perturbed scenarios; the
    result is a complete ZB-V program, the same on every call (ranks derive it independently), and
    not longer on the nominal costs than 3 % over the plain choice."""
    from elf_b200.scheduling.schedulers import generate_zbv_schedule
    from elf_b200.scheduling.simulator import simulate

    p, n = 4, 8
    placement = list(range(p)) + list(range(p - 1, -1, -1))
    costs = [(1.0 + 0.05 * s, 1.3 + 0.02 * s, 0.8) for s in range(2 * p)]
    costs[-1] = (1.6, 1.7, 1.5)
    which = {OperationType.FORWARD: 0, OperationType.BACKWARD_INPUTS: 1, OperationType.BACKWARD_PARAMS: 2}
    dur = lambda op: costs[op.block_id][which[op.op]] if op.op in which else 0.0
    plain = generate_zbv_schedule(placement, n, cap="auto", stage_costs=costs)
    a = generate_zbv_schedule(placement, n, cap="auto", stage_costs=costs, robust=0.02)
    b = generate_zbv_schedule(placement, n, cap="auto", stage_costs=costs, robust=0.02)
    assert [(o.op, o.block_id, o.mb_id, o.rank) for o in a] == [(o.op, o.block_id, o.mb_id, o.rank) for o in b]
    for kind in which:
        assert sorted((o.block_id, o.mb_id) for o in a if o.op == kind) == sorted((s, m) for s in range(2 * p) for m in range(n))
    assert simulate(a, placement, dur).makespan <= 1.03 * simulate(plain, placement, dur).makespan
