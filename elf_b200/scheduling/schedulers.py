"""The static schedule zoo.

Every generator has the signature ``(placement, n_micro_batches) -> List[Operation]`` and
returns the programs of **all** ranks, rank after rank (reference
``elf/scheduling/schedulers.py``; registry keys in ``elf/scheduling/__init__.py:11-66``).

Two construction styles are used:

* closed forms for the schedules whose per-rank program is a simple function of the
  rank's depth in the pipeline (GPipe, linear 1F1B, ZB-H1, ZB-H2, full-remat, inference);
* a policy-driven **list scheduler** (``_list_schedule``) that plays the pipeline forward
  in unit time steps and lets every idle rank pick its next op by priority
  (backward-inputs > forward under an in-flight cap > backward-params).  It produces
  interleaved 1F1B, Hanayo (any number of waves) and ZB-V for *any* number of
  micro-batches; the reference's ZB-V is a closed form valid only for
  ``nmb == 2 * n_devices`` (``elf/scheduling/schedulers.py:284-393``).

All generators work on the placement they are given with ranks taken relative to the
smallest rank in it, so a data-parallel replica offset cannot change the schedule
(the reference derives ``stages_per_device`` from ``max(placement)``,
``elf/scheduling/schedulers.py:52-54``, which breaks for shifted placements).
"""

from __future__ import annotations

import logging
from typing import Callable, Dict, List, Optional, Sequence

from .scheduling import Operation, OperationType, OpOptions

logger = logging.getLogger("schedulers")

__all__ = [
    "generate_afab_schedule",
    "generate_1f1b_schedule",
    "generate_hanayo_schedule",
    "generate_full_remat_schedule",
    "generate_zbh1_schedule",
    "generate_zbh2_schedule",
    "generate_zbv_schedule",
    "generate_inference_schedule",
    "FixedSchedule",
    "whole_stage_remat",
]

T = OperationType


def whole_stage_remat(name, _module=None) -> bool:
    """Remat strategy that checkpoints the stage as one unit (root module has name '')."""
    return name == ""


class _Programs:
    """Collects the per-rank programs and adds the loss ops around the last stage."""

    def __init__(self, placement: Sequence[int]):
        self.placement = list(placement)
        self.last = len(self.placement) - 1
        self.by_rank: Dict[int, List[Operation]] = {r: [] for r in sorted(set(self.placement))}

    def F(self, stage: int, mb: int, **opts) -> None:
        rank = self.placement[stage]
        prog = self.by_rank[rank]
        prog.append(Operation(stage, mb, T.FORWARD, rank, **opts))
        if stage == self.last:
            prog.append(Operation(stage, mb, T.LOSS_FORWARD, rank, **opts))

    def B(self, stage: int, mb: int, **opts) -> None:
        rank = self.placement[stage]
        prog = self.by_rank[rank]
        if stage == self.last:
            prog.append(Operation(stage, mb, T.LOSS_BACKWARD, rank, **opts))
        prog.append(Operation(stage, mb, T.BACKWARD_INPUTS, rank, **opts))

    def W(self, stage: int, mb: int, **opts) -> None:
        rank = self.placement[stage]
        self.by_rank[rank].append(Operation(stage, mb, T.BACKWARD_PARAMS, rank, **opts))

    def BW(self, stage: int, mb: int, **opts) -> None:
        self.B(stage, mb, **opts)
        self.W(stage, mb, **opts)

    def flat(self) -> List[Operation]:
        return [op for rank in self.by_rank for op in self.by_rank[rank]]


def _stages_by_rank(placement: Sequence[int]) -> Dict[int, List[int]]:
    out: Dict[int, List[int]] = {}
    for stage, rank in enumerate(placement):
        out.setdefault(rank, []).append(stage)
    return dict(sorted(out.items()))


# ---------------------------------------------------------------------------------------
# closed forms
# ---------------------------------------------------------------------------------------


def generate_afab_schedule(placement, n_micro_batches) -> List[Operation]:
    """GPipe: all forwards, then all backwards (B immediately followed by its W)."""
    out = _Programs(placement)
    for stages in _stages_by_rank(placement).values():
        for mb in range(n_micro_batches):
            for s in stages:
                out.F(s, mb)
        for mb in range(n_micro_batches):
            for s in reversed(stages):
                out.BW(s, mb)
    return out.flat()


def _is_linear(placement) -> bool:
    return len(set(placement)) == len(placement)


def generate_1f1b_schedule(placement, n_micro_batches) -> List[Operation]:
    """One-forward-one-backward.  One stage per rank: the classic PipeDream-flush program
    (``depth`` warm-up forwards, then B/W and F alternate, then the remaining B/W).
    Several stages per rank (``[0..p-1] * v``): interleaved 1F1B with ``(p-d-1) + (v-1)p``
    warm-up forwards at pipeline depth ``d`` when ``nmb`` is a multiple of ``p``; other
    shapes come from the list scheduler under the same in-flight bound."""
    n = n_micro_batches
    if _is_linear(placement):
        out = _Programs(placement)
        n_stages = len(placement)
        for s in range(n_stages):
            warm = min(n, n_stages - s)
            for mb in range(warm):
                out.F(s, mb)
            for i in range(n - warm):
                out.BW(s, i)
                out.F(s, warm + i)
            for mb in range(n - warm, n):
                out.BW(s, mb)
        return out.flat()

    ranks = sorted(set(placement))
    p = len(ranks)
    v = len(placement) // p
    by_rank = _stages_by_rank(placement)
    regular = n % p == 0 and all(len(st) == v for st in by_rank.values())
    if not regular:
        cap = {r: (p - d - 1) + (v - 1) * p + 1 for d, r in enumerate(ranks)}
        return _list_schedule(placement, n, split_w=False, cap=cap)

    # Virtual step k of a rank works on chunk (k // p) % v for forwards (mirrored for
    # backwards) and on micro-batch p * (k // (p v)) + k % p: groups of p micro-batches
    # sweep the chunks in turn.
    def fwd_step(k):
        return (k // p) % v, (k // (p * v)) * p + k % p

    def bwd_step(k):
        return v - 1 - (k // p) % v, (k // (p * v)) * p + k % p

    out = _Programs(placement)
    total = n * v
    for d, r in enumerate(ranks):
        stages = by_rank[r]
        warm = min(total, (p - d - 1) + (v - 1) * p)
        for k in range(warm):
            c, mb = fwd_step(k)
            out.F(stages[c], mb)
        for i in range(total - warm):
            c, mb = fwd_step(warm + i)
            out.F(stages[c], mb)
            c, mb = bwd_step(i)
            out.BW(stages[c], mb)
        for i in range(total - warm, total):
            c, mb = bwd_step(i)
            out.BW(stages[c], mb)
    return out.flat()


def generate_full_remat_schedule(placement, n_micro_batches) -> List[Operation]:
    """Every rank but the last runs GPipe with the whole stage checkpointed in F; the last
    rank runs F,B,W per micro-batch and keeps its activations."""
    out = _Programs(placement)
    by_rank = _stages_by_rank(placement)
    last_rank = max(by_rank)
    for rank, stages in by_rank.items():
        if rank == last_rank:
            for mb in range(n_micro_batches):
                for s in stages:
                    out.F(s, mb)
                for s in reversed(stages):
                    out.BW(s, mb)
            continue
        for mb in range(n_micro_batches):
            for s in stages:
                out.F(s, mb, **{OpOptions.REMAT_STRATEGY: whole_stage_remat})
        for mb in range(n_micro_batches):
            for s in reversed(stages):
                out.BW(s, mb)
    return out.flat()


def _zero_bubble_linear(placement, n, warm_of: Callable[[int, int], int], lag_of: Callable[[int, int, int], int]):
    """Shared shape of ZB-H1/ZB-H2 on a linear placement: ``warm`` forwards, one B, ``lag``
    rounds of (F, B) with no W, then rounds of (W, F, B) until everything is issued."""
    out = _Programs(placement)
    p = len(set(placement))
    for s in range(len(placement)):
        warm = warm_of(p, s)
        warm = min(n, warm)
        f = b = w = 0
        for _ in range(warm):
            out.F(s, f)
            f += 1
        out.B(s, b)
        b += 1
        for _ in range(lag_of(p, s, warm)):
            if f < n:
                out.F(s, f)
                f += 1
            if b < n:
                out.B(s, b)
                b += 1
        while f < n or b < n or w < n:
            if w < n:
                out.W(s, w)
                w += 1
            if f < n:
                out.F(s, f)
                f += 1
            if b < n:
                out.B(s, b)
                b += 1
    return out.flat()


def generate_zbh1_schedule(placement, n_micro_batches) -> List[Operation]:
    """ZB-H1: 1F1B's memory, W deferred by ``depth + 1`` backward slots.  The lag is the
    stage's depth in the pipeline (the reference uses the *global* rank,
    ``elf/scheduling/schedulers.py:223``, so replicas would disagree)."""
    return _zero_bubble_linear(placement, n_micro_batches, lambda p, s: p - s, lambda p, s, warm: s)


def generate_zbh2_schedule(placement, n_micro_batches) -> List[Operation]:
    """ZB-H2: ``2(p - s) - 1`` warm-up forwards; every W is pushed behind the 1F1B body
    so the tail bubble is filled with weight-gradient work."""
    n = n_micro_batches
    return _zero_bubble_linear(placement, n, lambda p, s: 2 * (p - s) - 1, lambda p, s, warm: max(0, n - 1 - warm))


def generate_inference_schedule(placement, n_micro_batches) -> List[Operation]:
    """Forward only; no loss ops."""
    sched = []
    for stage, rank in enumerate(placement):
        for mb in range(n_micro_batches):
            sched.append(Operation(stage, mb, T.FORWARD, rank))
    sched.sort(key=lambda op: op.rank)  # stable: rank after rank
    return sched


class FixedSchedule:
    """Replay ``{"order": [(kind, block_id, mb_id), ...]}`` with ``kind`` in ``f``/``b``/``w``
    (tuple order as emitted by the ILP and read by the reference,
    ``elf/scheduling/schedulers.py:408-440``)."""

    def __init__(self, schedule_dict):
        self.schedule_dict = schedule_dict

    def __call__(self, placement, n_micro_batches) -> List[Operation]:
        out = _Programs(placement)
        emit = {"f": out.F, "b": out.B, "w": out.W}
        for kind, block_id, mb_id in self.schedule_dict["order"]:
            emit[str(kind).lower()](int(block_id), int(mb_id))
        return out.flat()


# ---------------------------------------------------------------------------------------
# list scheduler
# ---------------------------------------------------------------------------------------


def _list_schedule(
    placement,
    n: int,
    *,
    split_w: bool,
    cap: Dict[int, int] | int | None = None,
    cost_f: float = 1,
    cost_b: float = 1,
    cost_w: float = 1,
    hop: float = 0,
    stage_costs: Optional[Sequence[float]] = None,
) -> List[Operation]:
    """Greedy event-driven simulation of the whole pipeline.

    Whenever a rank becomes idle it starts, in this order of preference,
    (1) the oldest ready backward-inputs (ready = own forward done and the next stage's B
        done, ``hop`` later when that stage is on another rank);
    (2) the deepest ready forward, if the rank holds fewer than ``cap`` live
        (stage, micro-batch) activations (live = forwarded, W not yet run);
    (3) the oldest pending backward-params (only when ``split_w``; otherwise W is glued
        to its B);
    otherwise it idles until the next completion anywhere in the pipeline.  An op of stage
    ``s`` lasts ``stage_costs[s]`` (default 1) times ``cost_f`` / ``cost_b`` / ``cost_w``, so
    stages of unequal weight (more layers, the LM head) and F/B/W of unequal length are
    scheduled for what they cost rather than as unit slots.  If the cap ever starves the
    whole pipeline it is lifted by one on the blocked ranks.  Because the result is read
    off a feasible timeline, the per-rank programs admit a global order and cannot
    deadlock once comms are added.
    """
    n_stages = len(placement)
    by_rank = _stages_by_rank(placement)
    ranks = list(by_rank)
    if cap is None:
        cap = {r: n_stages * n for r in ranks}
    elif isinstance(cap, int):
        cap = {r: cap for r in ranks}
    cap = dict(cap)
    if stage_costs is None:
        stage_costs = [1.0] * n_stages
    assert len(stage_costs) == n_stages, "one cost per stage"
    # an entry is either a relative weight (multiplied by cost_f / cost_b / cost_w) or a measured
    # (forward, backward-inputs, backward-params) triple of durations that is taken as it is
    dur_f, dur_b, dur_w = [], [], []
    for c in stage_costs:
        if isinstance(c, (tuple, list)):
            f, b, w = (float(x) for x in c)
        else:
            f, b, w = cost_f * float(c), cost_b * float(c), cost_w * float(c)
        dur_f.append(f)
        dur_b.append(b)
        dur_w.append(w)

    UNSET = None
    f_end: List[List[Optional[float]]] = [[UNSET] * n for _ in range(n_stages)]
    b_end: List[List[Optional[float]]] = [[UNSET] * n for _ in range(n_stages)]
    f_next = [0] * n_stages
    b_next = [0] * n_stages
    w_next = [0] * n_stages
    free_at = {r: 0.0 for r in ranks}
    out = _Programs(placement)
    total = n_stages * n * 3
    done = 0
    EPS = 1e-9

    def arrival(end: float, src_stage: int, dst_stage: int) -> float:
        return end + (hop if placement[src_stage] != placement[dst_stage] else 0)

    def f_ready_at(s: int) -> Optional[float]:
        """Time from which the next forward of stage ``s`` may start (None: not yet known)."""
        mb = f_next[s]
        if mb >= n:
            return None
        if s == 0:
            return 0.0
        e = f_end[s - 1][mb]
        return None if e is UNSET else arrival(e, s - 1, s)

    def b_ready_at(s: int) -> Optional[float]:
        mb = b_next[s]
        if mb >= n or f_end[s][mb] is UNSET:
            return None
        t0 = f_end[s][mb]
        if s == n_stages - 1:
            return t0
        e = b_end[s + 1][mb]
        return None if e is UNSET else max(t0, arrival(e, s + 1, s))

    def live(rank: int) -> int:
        return sum(f_next[s] - w_next[s] for s in by_rank[rank])

    stalled_rounds = 0
    while done < total:
        r = min(ranks, key=lambda q: (free_at[q], q))
        t = free_at[r]
        stages = by_rank[r]
        b_times = {s: b_ready_at(s) for s in stages}
        cand_b = [s for s in stages if b_times[s] is not None and b_times[s] <= t + EPS]
        if cand_b:
            s = min(cand_b, key=lambda s: (b_next[s], s))
            mb = b_next[s]
            out.B(s, mb)
            b_next[s] += 1
            dur = dur_b[s]
            done += 1
            b_end[s][mb] = t + dur
            if not split_w:
                out.W(s, mb)
                w_next[s] += 1
                dur += dur_w[s]
                done += 1
            free_at[r] = t + dur
            stalled_rounds = 0
            continue
        f_times = {s: f_ready_at(s) for s in stages}
        cand_f = [s for s in stages if f_times[s] is not None and f_times[s] <= t + EPS]
        capped = bool(cand_f) and live(r) >= cap[r]
        if cand_f and not capped:
            s = max(cand_f, key=lambda s: (s, -f_next[s]))
            mb = f_next[s]
            out.F(s, mb)
            f_next[s] += 1
            f_end[s][mb] = t + dur_f[s]
            free_at[r] = f_end[s][mb]
            done += 1
            stalled_rounds = 0
            continue
        if split_w:
            cand_w = [s for s in stages if w_next[s] < b_next[s]]
            if cand_w:
                s = min(cand_w, key=lambda s: (w_next[s], s))
                out.W(s, w_next[s])
                w_next[s] += 1
                free_at[r] = t + dur_w[s]
                done += 1
                stalled_rounds = 0
                continue
        # nothing to do now: sleep until something this rank waits for can have happened
        known = [x for x in list(b_times.values()) + ([] if capped else list(f_times.values())) if x is not None and x > t + EPS]
        others = [free_at[q] for q in ranks if q != r and free_at[q] > t + EPS]
        wake = min(known + others) if (known or others) else None
        if wake is None:
            # every rank is idle at time t and nothing is in flight
            stalled_rounds += 1
            if stalled_rounds > len(ranks):
                blocked = [q for q in ranks if live(q) >= cap[q] and any(f_ready_at(s) is not None for s in by_rank[q])]
                if not blocked:
                    raise RuntimeError("list scheduler stalled: placement admits no feasible order")
                for q in blocked:
                    cap[q] += 1
                stalled_rounds = 0
            free_at[r] = t + EPS * 10  # let the other idle ranks be examined
        else:
            free_at[r] = wake
    return out.flat()


def generate_hanayo_schedule(placement, n_micro_batches) -> List[Operation]:
    """Hanayo wave schedule on ``[0..p-1, p-1..0] * waves``: forwards and (B, W) pairs are
    interleaved across the legs of each wave; every rank keeps at most ``p`` live
    micro-batches per local stage."""
    p = len(set(placement))
    return _list_schedule(placement, n_micro_batches, split_w=False, cap=max(1, len(placement) // p) * p)


def generate_zbv_schedule(placement, n_micro_batches, *, cap=None, stage_costs: Optional[Sequence[float]] = None,
                          ratios: Sequence[float] = (1.0, 1.0, 1.0), cap_limit: Optional[int] = None, robust: float = 0.0) -> List[Operation]:
    """ZB-V on the V placement ``[0..p-1, p-1..0]`` for any number of micro-batches.  Each
    rank holds at most ``cap`` live (stage, micro-batch) activations (default ``2p``, the
    footprint of 1F1B) and weight-gradient passes fill what would otherwise be bubbles.
    ``stage_costs`` (relative weight of every stage) and ``ratios`` (F : B : W durations)
    let the schedule be laid out for stages of unequal weight; use
    ``functools.partial(generate_zbv_schedule, stage_costs=...)`` as the scheduler.  An entry
    of ``stage_costs`` may also be a measured ``(forward, backward-inputs, backward-params)``
    triple of durations (see ``Pipeline.measured_stage_costs``); ``ratios`` is then ignored
    for that stage.

    ``cap="auto"`` lays the schedule out for several caps between ``2p`` and ``cap_limit``
    (default ``6p``), runs each through the timeline simulator with the same costs and keeps
    the shortest one (the smaller cap on ties): with a greedy list scheduler more live
    activations do not always give a shorter step, so the cap is chosen by measurement.

    ``robust`` (with ``cap="auto"``; a relative standard deviation such as 0.02): the greedy
    layout is tuned to the exact durations it is given, and measured durations move by a
    percent or two from step to step (per rank, as clocks drift under the power limit, and
    per stage).  With ``robust > 0`` candidates are also laid out for a few perturbed copies
    of the costs, and every candidate is scored by its mean simulated step over the nominal
    costs and several perturbed ones, so the schedule that is kept is one that stays short
    when the costs are a little off.  The perturbations come from a fixed seed: every rank
    derives the same schedule.  (Replayed on the durations measured later in the same runs,
    schedules chosen this way were 1-2 % shorter on 4 GPUs: 747 ms against 763 ms, 739 against
    747.)"""
    p = len(set(placement))
    if len(placement) != 2 * p:
        logger.warning("zbv expects a V placement with two stages per rank, got %s", list(placement))
    cf, cb, cw = ratios

    def build(c):
        return _list_schedule(placement, n_micro_batches, split_w=True, cap=c, cost_f=cf, cost_b=cb, cost_w=cw, stage_costs=stage_costs)

    if cap != "auto":
        return build(cap if cap is not None else 2 * p)
    from .simulator import simulate

    costs = list(stage_costs) if stage_costs is not None else [1.0] * len(placement)
    which = {OperationType.FORWARD: 0, OperationType.BACKWARD_INPUTS: 1, OperationType.BACKWARD_PARAMS: 2}

    def duration(op):
        k = which.get(op.op)
        if k is None:
            return 0.0
        c = costs[op.block_id]
        return float(c[k]) if isinstance(c, (tuple, list)) else float(c) * (cf, cb, cw)[k]

    limit = cap_limit if cap_limit is not None else 6 * p
    candidates = sorted({c for c in (2 * p, (5 * p) // 2, 3 * p, (7 * p) // 2, 4 * p, 5 * p, 6 * p, limit) if 2 <= c <= limit})
    if robust > 0.0:
        return _robust_zbv(placement, n_micro_batches, costs, (cf, cb, cw), candidates, robust)
    best = None
    for c in candidates:
        sched = build(c)
        span = simulate(sched, list(placement), duration).makespan
        if best is None or span < best[0] * (1.0 - 1e-6):
            best = (span, c, sched)
    logger.info("zbv: cap %d of %s chosen (simulated makespan %.2f)", best[1], candidates, best[0])
    return best[2]


def _robust_zbv(placement, n_micro_batches, costs, ratios, caps, sigma: float, n_layouts: int = 8, n_scenarios: int = 12) -> List[Operation]:
    """Lay ZB-V out for the nominal costs and ``n_layouts - 1`` perturbed copies of them, for every
    cap, and keep the layout whose simulated step, averaged over the nominal costs and
    ``n_scenarios`` perturbed ones, is the shortest.  A perturbation scales every rank by
    ``N(1, sigma)`` and every stage by ``N(1, sigma / 2)`` on top (seeded: the same on all ranks)."""
    import random

    from .simulator import simulate

    placement = list(placement)
    triples = [tuple(float(x) for x in c) if isinstance(c, (tuple, list)) else tuple(float(c) * r for r in ratios) for c in costs]
    which = {OperationType.FORWARD: 0, OperationType.BACKWARD_INPUTS: 1, OperationType.BACKWARD_PARAMS: 2}
    rng = random.Random(20240229)
    ranks = sorted(set(placement))

    def perturbed():
        by_rank = {r: 1.0 + rng.gauss(0.0, sigma) for r in ranks}
        return [tuple(v * by_rank[placement[s]] * (1.0 + rng.gauss(0.0, sigma / 2)) for v in t) for s, t in enumerate(triples)]

    scenarios = [triples] + [perturbed() for _ in range(n_scenarios)]
    layouts = [triples] + [perturbed() for _ in range(n_layouts - 1)]
    best = None
    for k, layout in enumerate(layouts):
        for c in caps:
            sched = _list_schedule(placement, n_micro_batches, split_w=True, cap=c, stage_costs=layout)
            score = 0.0
            for scenario in scenarios:
                score += simulate(sched, placement, lambda op: scenario[op.block_id][which[op.op]] if op.op in which else 0.0).makespan
            score /= len(scenarios)
            if best is None or score < best[0] * (1.0 - 1e-6):
                best = (score, c, k, sched)
    logger.info("zbv: cap %d, layout %d of %d chosen (mean simulated makespan %.4g over %d cost scenarios)", best[1], best[2], len(layouts), best[0], len(scenarios))
    return best[3]
