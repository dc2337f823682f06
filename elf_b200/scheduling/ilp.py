"""Rematerialisation (and offload) under a per-GPU memory budget, chosen by an ILP.

Pipeline of this module (reference ``elf/scheduling/ilp.py``):

1. **profile** every stage: time of F / B / W (ms), memory kept after each (MB), transient
   peaks, checkpointed-forward peak, bytes of split-backward stashes, input/output sizes,
   and the p2p time of the stage's output (``profile_all_stages``; statistics schema of
   ``profile`` in the reference, ``:158-206``);
2. **solve** a mixed-integer program over one binary per (stage, micro-batch, option) and
   continuous end times per op: minimise the makespan subject to data-flow precedence
   (with communication time across ranks), the per-rank program order of a base schedule,
   a memory bound at every program position, and at most one forward-side and one
   backward-side option per (stage, micro-batch) — constraint set of the reference's
   ``solve_remat`` (``:491-747``).  Options: ``full_fwd`` (checkpoint the stage in F, pay
   T_f at B), ``activations_bwd`` (drop W-pass inputs after B, pay T_f before W),
   ``full_bwd`` (drop them and the output-grads, pay T_f + T_b before W) and, new here,
   ``offload`` (park the forward's saved activations in pinned host memory; pays only the
   part of the PCIe copy that cannot be hidden, and the total copy time per rank is
   bounded by the makespan);
3. **apply** the solution to the base schedule (``RematScheduler``), solving on one rank and
   broadcasting the result (``stagerematify``), or doing so for every base schedule and
   keeping the fastest (``AutoScheduler``).

The program is solved with ``scipy.optimize.milp`` (HiGHS), which ships with this
environment; the reference needs the external ``pulp`` package and a CBC/CPLEX binary.
Budgets are in MB, as in the reference.  Works on CPU (memory is then estimated from the
tensors autograd saves) so that the whole path is testable without a GPU.
"""

from __future__ import annotations

import logging
import statistics as _stats
import time
from dataclasses import dataclass
from typing import Callable, Dict, List, Optional, Sequence, Tuple

import torch
import torch.distributed as dist
from torch.utils.checkpoint import checkpoint

from ..partitioners.signature import Signature
from ..registry import SCHEDULERS, resolve
from ..utils.metadata import TensorMetadata
from ..utils.timers import Timer
from ..zb_utils import LayerDW
from .offload_sched import apply_offload
from .scheduling import Operation, OperationType, OpOptions

logger = logging.getLogger("elf.ilp")

__all__ = [
    "profile",
    "profile_stage",
    "profile_all_stages",
    "propagate_sample",
    "profile_communication",
    "build_ilp_params",
    "solve_remat",
    "RematOption",
    "RematScheduler",
    "stagerematify",
    "AutoScheduler",
    "init_tensor_",
]

_MB = 1024 * 1024
T = OperationType


# =======================================================================================
# 1. profiling
# =======================================================================================


def _on_cuda(stage: torch.nn.Module) -> bool:
    return any(p.is_cuda for p in stage.parameters())


class _SavedBytes:
    """Counts bytes of distinct storages saved by autograd (memory estimate on CPU)."""

    def __init__(self):
        self.seen: Dict[int, int] = {}

    def __enter__(self):
        def pack(t):
            if isinstance(t, torch.Tensor) and not isinstance(t, torch.nn.Parameter):
                st = t.untyped_storage()
                self.seen[st.data_ptr()] = st.nbytes()
            return t

        self._ctx = torch.autograd.graph.saved_tensors_hooks(pack, lambda t: t)
        self._ctx.__enter__()
        return self

    def __exit__(self, *exc):
        self._ctx.__exit__(*exc)
        return False

    @property
    def mb(self) -> float:
        return sum(self.seen.values()) / _MB


def _bparams(stage: torch.nn.Module) -> None:
    for m in stage.modules():
        if isinstance(m, LayerDW):
            m.move_last_computed("input", 0)
            m.move_last_computed("grad_output", 0)
            if len(m.ctx["grad_output"]) > 0 and m.ctx["grad_output"][0] is not None and m.ctx["input"][0] is not None:
                m.backward(0)
            m.clear()


def _fake_loss(outputs) -> torch.Tensor:
    return sum(o.float().sum() for o in outputs if isinstance(o, torch.Tensor) and o.requires_grad)


def _stash_bytes(stage: torch.nn.Module, attr: str) -> float:
    total = 0
    for m in stage.modules():
        if isinstance(m, LayerDW):
            t = getattr(m, attr, None)
            if t is not None:
                total += t.nbytes
    return total / _MB


def _measure_full_pass(stage: torch.nn.Module, sample: Sequence[torch.Tensor], n_iter: int = 3):
    """``(T, M, Mpeak, Minput, Moutput, Mbg, warm-up outputs)`` for one stage; times in ms,
    memories in MB relative to the state before the forward."""
    cuda = _on_cuda(stage)
    dev = next(stage.parameters()).device if cuda else None

    def sync():
        if cuda:
            torch.cuda.synchronize(dev)

    def leafs():
        return tuple(s.detach().requires_grad_(s.is_floating_point() or s.is_complex()) for s in sample)

    def run_forward():
        out = stage(*leafs())
        return out if isinstance(out, tuple) else (out,)

    outs = run_forward()
    warm = tuple(o.detach() for o in outs if isinstance(o, torch.Tensor))
    loss = _fake_loss(outs)
    if isinstance(loss, torch.Tensor):
        loss.backward()
    _bparams(stage)
    del outs, loss
    sync()

    times = {k: [] for k in "fbw"}
    mems = {k: [] for k in "fbw"}
    peaks = {k: [] for k in "fbw"}
    mbg_samples = []
    minput = sum(s.nbytes for s in sample) / _MB
    moutput = sum(o.nbytes for o in warm) / _MB
    for _ in range(n_iter):
        stage.zero_grad(set_to_none=True)
        sync()
        if cuda:
            torch.cuda.reset_peak_memory_stats(dev)
            base = torch.cuda.memory_allocated(dev)
        saved = _SavedBytes()
        with Timer(name="f") as tf, saved:
            outs = run_forward()
            loss = _fake_loss(outs)
        times["f"].append(tf.time() * 1e3)
        if cuda:
            mems["f"].append((torch.cuda.memory_allocated(dev) - base) / _MB)
            peaks["f"].append((torch.cuda.max_memory_allocated(dev) - base) / _MB)
            torch.cuda.reset_peak_memory_stats(dev)
            before = torch.cuda.memory_allocated(dev)
        else:
            mf = saved.mb + moutput
            mems["f"].append(mf)
            peaks["f"].append(mf * 1.1)
        with Timer(name="b") as tb:
            if isinstance(loss, torch.Tensor):
                loss.backward()
            del outs, loss
        times["b"].append(tb.time() * 1e3)
        mba = _stash_bytes(stage, "last_input")
        mbg = _stash_bytes(stage, "last_grad_output")
        mbg_samples.append(mbg)
        if cuda:
            mems["b"].append((torch.cuda.memory_allocated(dev) - base) / _MB)
            peaks["b"].append((torch.cuda.max_memory_allocated(dev) - before) / _MB)
            torch.cuda.reset_peak_memory_stats(dev)
            before = torch.cuda.memory_allocated(dev)
        else:
            mems["b"].append(mba + mbg)
            peaks["b"].append(max(0.0, mems["f"][-1] * 0.5))
        with Timer(name="w") as tw:
            _bparams(stage)
        times["w"].append(tw.time() * 1e3)
        if cuda:
            mems["w"].append((torch.cuda.memory_allocated(dev) - base) / _MB)
            peaks["w"].append((torch.cuda.max_memory_allocated(dev) - before) / _MB)
        else:
            mems["w"].append(0.0)
            peaks["w"].append(0.0)
    stage.zero_grad(set_to_none=True)
    med = lambda d: {k: float(_stats.median(v)) for k, v in d.items()}
    return med(times), med(mems), med(peaks), minput, moutput, float(_stats.median(mbg_samples)), warm


def _measure_ckpt_forward(stage: torch.nn.Module, sample: Sequence[torch.Tensor]) -> Tuple[float, float]:
    """Peak of a fully checkpointed forward and the bytes of W-pass input stashes (MB)."""
    cuda = _on_cuda(stage)
    dev = next(stage.parameters()).device if cuda else None
    leafs = tuple(s.detach().requires_grad_(s.is_floating_point() or s.is_complex()) for s in sample)
    if cuda:
        torch.cuda.synchronize(dev)
        torch.cuda.reset_peak_memory_stats(dev)
        base = torch.cuda.memory_allocated(dev)
    out = checkpoint(stage, *leafs, use_reentrant=False)
    if cuda:
        torch.cuda.synchronize(dev)
        peak = (torch.cuda.max_memory_allocated(dev) - base) / _MB
    else:
        outs = out if isinstance(out, tuple) else (out,)
        peak = sum(o.nbytes for o in outs if isinstance(o, torch.Tensor)) / _MB * 2 + sum(s.nbytes for s in sample) / _MB
    mba = _stash_bytes(stage, "last_input")
    for m in stage.modules():
        if isinstance(m, LayerDW):
            m.clear()
    del out
    return float(peak), float(mba)


def init_tensor_(t: torch.Tensor, int_high: int = 100) -> torch.Tensor:
    """Random fill by dtype: N(0,1) for floats, uniform ``[0, int_high)`` for integers."""
    if t.is_floating_point() or t.is_complex():
        t.normal_(0.0, 1.0)
    elif t.dtype == torch.bool:
        t.random_(0, 2)
    else:
        t.random_(0, int_high)
    return t


def _stats_dict(stage, T_, M_, Mpeak, minput, moutput, mbg, peak_ckpt, mba, tcomm=0.0) -> dict:
    return {
        "T": T_,
        "M": M_,
        "Mpeak": Mpeak,
        "Mpeak_ckpt": peak_ckpt,
        "Mparams": sum(p.nbytes for p in stage.parameters()) / _MB,
        "Mba": mba,
        "Mbg": mbg if mbg > 0 else max(0.0, M_["b"] - mba),
        "Minput": minput,
        "Moutput": moutput,
        "Tcomm": tcomm,
        "forward_remat_options": [],
        "backward_remat_options": [],
    }


def profile_stage(stage: torch.nn.Module, sample_metadata, n_iter: int = 10, sample: Optional[Sequence[torch.Tensor]] = None):
    """Statistics of one stage (no communication) and the outputs of its warm-up forward.
    ``sample_metadata`` is a sequence of ``TensorMetadata`` whose shapes include the
    micro-batch dimension; a concrete ``sample`` overrides the random fill."""
    if sample is None:
        sample = tuple(init_tensor_(m.get_buffer(1).squeeze(0)) for m in sample_metadata)
    T_, M_, Mpeak, minput, moutput, mbg, warm = _measure_full_pass(stage, sample, n_iter)
    peak_ckpt, mba = _measure_ckpt_forward(stage, sample)
    return _stats_dict(stage, T_, M_, Mpeak, minput, moutput, mbg, peak_ckpt, mba), warm


def _measure_communication(signature: Signature, minput: float, moutput: float, placement, my_rank: int, to_global: Callable[[int], int], device, n_iter: int = 20, group=None) -> float:
    """Median ms of a blocking send of this stage's output to its consumer (0 when local).
    Every rank calls this for its own stages in stage order, so sends meet their recvs."""
    for src in signature.sources:
        if src is None or placement[src] == my_rank:
            continue
        buf = torch.empty(max(1, int(minput * _MB) // 4), dtype=torch.float32, device=device)
        for _ in range(n_iter):
            dist.recv(buf, to_global(placement[src]), group=group)
    samples = []
    for tgt in signature.targets:
        t = tgt[0] if tgt else None
        if t is None or placement[t] == my_rank:
            samples.append(0.0)
            continue
        buf = torch.empty(max(1, int(moutput * _MB) // 4), dtype=torch.float32, device=device)
        for _ in range(n_iter):
            with Timer(name="comm") as tm:
                dist.send(buf, to_global(placement[t]), group=group)
            samples.append(tm.time() * 1e3)
    return float(_stats.median(samples)) if samples else 0.0


def profile(stages: List[torch.nn.Module], samples: List[Sequence[torch.Tensor]], signatures: List[Signature], placement: List[int]) -> List[dict]:
    """Stand-alone profiling of a list of stages held by this process (communication time
    is measured only when ``torch.distributed`` is up).  One dictionary per stage:

    ``T`` {f,b,w} ms · ``M`` {f,b,w} MB kept after the op · ``Mpeak`` {f,b,w} MB transient ·
    ``Mpeak_ckpt`` · ``Mparams`` · ``Mba`` (W-pass input stashes) · ``Mbg`` (output-grad
    stashes) · ``Minput`` · ``Moutput`` · ``Tcomm`` ms."""
    out = []
    for stage, sample, sig in zip(stages, samples, signatures):
        sample = tuple(sample) if isinstance(sample, (tuple, list)) else (sample,)
        st, _ = profile_stage(stage, None, n_iter=3, sample=sample)
        out.append(st)
    return out


def _drop_fake_caches(model: torch.nn.Module) -> None:
    """Modules may cache tensors they compute on first use (rotary tables, masks).  A cache filled
    during the shape-propagation pass holds fake tensors; left in place, later real forwards would
    compute on them and hand fake outputs to the transport.  Reset such attributes to ``None``."""
    from torch._subclasses.fake_tensor import FakeTensor

    def is_fake(v) -> bool:
        if isinstance(v, FakeTensor):
            return True
        if isinstance(v, (tuple, list)):
            return any(is_fake(x) for x in v)
        if isinstance(v, dict):
            return any(is_fake(x) for x in v.values())
        return False

    for m in model.modules():
        for name, value in list(vars(m).items()):
            if name.startswith("_parameters") or name in ("_buffers", "_modules"):
                continue
            if is_fake(value):
                setattr(m, name, None)


def propagate_sample(block_models: Dict[int, torch.nn.Module], placement, sample, pp_group, to_global: Callable[[int], int] = lambda r: r, my_rank: Optional[int] = None):
    """Input metadata of every local block, found by running the blocks on ``meta`` copies
    of their inputs stage after stage; at rank boundaries only the shapes travel (as a
    pickled list).  Returns ``{block id: (TensorMetadata, ...)}`` with full shapes."""
    from torch._subclasses.fake_tensor import FakeTensorMode

    if my_rank is None:
        my_rank = dist.get_rank() if dist.is_initialized() else 0
    sample = tuple(sample) if isinstance(sample, (tuple, list)) else (sample,)
    metas: Dict[int, tuple] = {}
    out_meta = None
    mode = FakeTensorMode(allow_non_fake_inputs=True)
    for block_id in range(len(placement)):
        owner = placement[block_id]
        prev = placement[block_id - 1] if block_id else None
        if owner == my_rank:
            if block_id == 0:
                in_meta = tuple(TensorMetadata(shape=list(s.shape), dtype=s.dtype) for s in sample)
            elif prev == my_rank:
                in_meta = out_meta
            else:
                box = [None]
                dist.recv_object_list(box, src=to_global(prev), group=pp_group)
                in_meta = tuple(TensorMetadata(shape=s, dtype=d) for s, d in box[0])
            metas[block_id] = in_meta
            model = block_models[block_id]
            dev = next(model.parameters()).device if any(True for _ in model.parameters()) else torch.device("cpu")
            with mode, torch.no_grad():
                fake_in = tuple(torch.empty(m.shape, dtype=m.dtype, device=dev) for m in in_meta)
                fake_out = model(*fake_in)
            fake_out = fake_out if isinstance(fake_out, tuple) else (fake_out,)
            out_meta = tuple(TensorMetadata(shape=list(o.shape), dtype=o.dtype) for o in fake_out)
            for m in model.modules():
                if isinstance(m, LayerDW):
                    m.clear()
            _drop_fake_caches(model)
        elif prev == my_rank and block_id:
            dist.send_object_list([[(m.shape, m.dtype) for m in out_meta]], dst=to_global(owner), group=pp_group)
    return metas


def profile_communication(local_stats: Dict[int, dict], signatures, placement, pp_group, my_rank: int, to_global, device) -> None:
    for block_id in sorted(local_stats):
        st = local_stats[block_id]
        st["Tcomm"] = _measure_communication(signatures[block_id], st["Minput"], st["Moutput"], list(placement), my_rank, to_global, device, group=pp_group)


def profile_all_stages(blocks, signatures, placement, sample, pp_group) -> List[dict]:
    """Every pipeline rank profiles its own stages, then the dictionaries are gathered
    over the pipeline group.  Returns one entry per stage, in stage order."""
    distributed = dist.is_available() and dist.is_initialized() and pp_group is not None and dist.get_world_size(pp_group) > 1
    my_rank = blocks[0].rank if blocks else 0
    if distributed:
        members = dist.get_process_group_ranks(pp_group)
        to_global = lambda r: members[r]
    else:
        to_global = lambda r: r
    models = {b.id: b.model for b in blocks}
    if distributed:
        metas = propagate_sample(models, placement, sample, pp_group, to_global, my_rank)
    else:
        metas = {}
        cur = tuple(sample) if isinstance(sample, (tuple, list)) else (sample,)
    local: Dict[int, dict] = {}
    for block in sorted(blocks, key=lambda b: b.id):
        if distributed:
            dev = block.device
            smp = tuple(init_tensor_(torch.empty(m.shape, dtype=m.dtype, device=dev)) for m in metas[block.id])
        else:
            smp = tuple(t.to(block.device) for t in cur)
        st, warm = profile_stage(block.model, None, n_iter=5, sample=smp)
        cur = warm
        block.model.zero_grad(set_to_none=True)
        for layer in block.dw_layers():
            layer.clear()
        if block.device.type == "cuda":
            torch.cuda.empty_cache()
        local[block.id] = st
    if not distributed:
        return [local[i] for i in range(len(placement))]
    profile_communication(local, signatures, placement, pp_group, my_rank, to_global, blocks[0].device if blocks else torch.device("cpu"))
    gathered = [None] * dist.get_world_size(pp_group)
    dist.all_gather_object(gathered, local, group=pp_group)
    out: List[Optional[dict]] = [None] * len(placement)
    for d in gathered:
        for block_id, st in (d or {}).items():
            out[block_id] = st
    return out


# =======================================================================================
# 2. the mixed-integer program
# =======================================================================================


@dataclass
class RematOption:
    name: str
    type: str  # "forward" or "backward"
    mem_freed: float  # MB
    time_overhead: float  # ms


_OP_INDEX = {"f": 0, "b": 1, "w": 2}
_LETTER = {T.FORWARD: "f", T.BACKWARD_INPUTS: "b", T.BACKWARD_PARAMS: "w"}


def _simplified(placement, nmb, scheduler) -> List[List[Tuple[str, int, int]]]:
    ranks = sorted(set(placement))
    index = {r: i for i, r in enumerate(ranks)}
    out: List[List[Tuple[str, int, int]]] = [[] for _ in ranks]
    for op in scheduler(placement, nmb):
        if op.op in _LETTER:
            out[index[op.rank]].append((_LETTER[op.op], op.block_id, op.mb_id))
    return out


def build_ilp_params(statistics, placement, scheduler, n_micro_batches, memory_budget, offload: bool = False, pcie_gbs: float = 50.0, offload_overlap: float = 0.85) -> dict:
    """Plain-data description of the problem (stage costs, option tables, per-rank order)."""
    nstages = len(placement)
    assert len(statistics) == nstages, "one statistics entry per stage"
    stages = []
    for st in statistics:
        T_, M_ = st["T"], st["M"]
        act = max(0.0, M_["f"] - st["Minput"] - st["Moutput"])
        fwd = [RematOption("full_fwd", "forward", act, T_["f"])]
        if offload:
            copy_ms = act / 1024.0 / pcie_gbs * 1e3  # one direction
            fwd.append(RematOption("offload", "forward", act, 2 * copy_ms * (1.0 - offload_overlap)))
        bwd = [
            RematOption("activations_bwd", "backward", st["Mba"], T_["f"]),
            RematOption("full_bwd", "backward", max(0.0, M_["b"] - st["Moutput"] - st["Minput"]), T_["f"] + T_["b"]),
        ]
        peaks = dict(st["Mpeak"])
        peaks["f_no_grad"] = st["Mpeak_ckpt"]
        stages.append({"T": T_, "M": M_, "Mpeak": peaks, "Tcomm": st["Tcomm"], "Mparams": st["Mparams"], "act": act,
                       "fwd_remat_options": fwd, "bwd_remat_options": bwd})
    return {
        "p": len(set(placement)),
        "m": n_micro_batches,
        "nstages": nstages,
        "MGpu": memory_budget,
        "sched": _simplified(placement, n_micro_batches, scheduler),
        "placement": list(placement),
        "stages": stages,
        "pcie_gbs": pcie_gbs,
    }


class _LinExpr:
    """Sparse affine expression ``const + Σ coef·var`` used to assemble the constraint matrix."""

    __slots__ = ("c", "t")

    def __init__(self, const: float = 0.0, terms: Optional[Dict[int, float]] = None):
        self.c = float(const)
        self.t = dict(terms) if terms else {}

    def add(self, other, scale: float = 1.0) -> "_LinExpr":
        if isinstance(other, _LinExpr):
            self.c += scale * other.c
            for k, v in other.t.items():
                self.t[k] = self.t.get(k, 0.0) + scale * v
        else:
            self.c += scale * float(other)
        return self

    def copy(self) -> "_LinExpr":
        return _LinExpr(self.c, self.t)

    def value(self, x) -> float:
        return self.c + sum(v * x[k] for k, v in self.t.items())


class _Program:
    def __init__(self):
        self.lb: List[float] = []
        self.ub: List[float] = []
        self.integer: List[int] = []
        self.rows: List[Tuple[Dict[int, float], float, float]] = []

    def var(self, lb=0.0, ub=float("inf"), integer=False) -> int:
        self.lb.append(lb)
        self.ub.append(ub)
        self.integer.append(1 if integer else 0)
        return len(self.lb) - 1

    def leq(self, expr: _LinExpr, rhs: float = 0.0) -> None:
        """expr <= rhs"""
        self.rows.append((expr.t, -float("inf"), rhs - expr.c))

    def geq(self, expr: _LinExpr, rhs: float = 0.0) -> None:
        self.rows.append((expr.t, rhs - expr.c, float("inf")))

    def eq(self, expr: _LinExpr, rhs: float = 0.0) -> None:
        self.rows.append((expr.t, rhs - expr.c, rhs - expr.c))

    def solve(self, objective: _LinExpr, time_limit: float, gap: float):
        import numpy as np
        from scipy.optimize import Bounds, LinearConstraint, milp
        from scipy.sparse import csr_matrix

        n = len(self.lb)
        c = np.zeros(n)
        for k, v in objective.t.items():
            c[k] = v
        data, ri, ci, lo, hi = [], [], [], [], []
        for r, (terms, l, h) in enumerate(self.rows):
            for k, v in terms.items():
                if v != 0.0:
                    data.append(v)
                    ri.append(r)
                    ci.append(k)
            lo.append(l)
            hi.append(h)
        A = csr_matrix((data, (ri, ci)), shape=(len(self.rows), n))
        res = milp(c, constraints=LinearConstraint(A, np.array(lo), np.array(hi)), integrality=np.array(self.integer),
                   bounds=Bounds(np.array(self.lb), np.array(self.ub)), options={"time_limit": float(time_limit), "mip_rel_gap": float(gap), "disp": False})
        return res


def solve_remat(statistics: List[dict], placement: List[int], scheduler, n_micro_batches: int, memory_budget: float, time_limit: int = 60, gap_rel_limit: float = 0.03, offload: bool = False, pcie_gbs: float = 50.0) -> dict:
    """Minimise the makespan of ``scheduler``'s program under ``memory_budget`` MB per rank.

    Returns ``{placement, objective (ms), peak_mems [MB per rank], order [(f|b|w, stage, mb)],
    full_fwd[stage][mb], activations_bwd[...], full_bwd[...], offload[...] (when enabled)}``.
    Raises ``RuntimeError`` when no assignment fits the budget."""
    prm = build_ilp_params(statistics, placement, scheduler, n_micro_batches, memory_budget, offload=offload, pcie_gbs=pcie_gbs)
    p, m, nstages, MGpu = prm["p"], prm["m"], prm["nstages"], prm["MGpu"]
    sched, stages, plc = prm["sched"], prm["stages"], prm["placement"]
    ranks = sorted(set(plc))
    rank_index = {r: i for i, r in enumerate(ranks)}
    on_rank = {i: [s for s, r in enumerate(plc) if rank_index[r] == i] for i in range(p)}

    prog = _Program()
    fwd = [[{o.name: prog.var(0, 1, True) for o in stages[s]["fwd_remat_options"]} for _ in range(m)] for s in range(nstages)]
    bwd = [[{o.name: prog.var(0, 1, True) for o in stages[s]["bwd_remat_options"]} for _ in range(m)] for s in range(nstages)]
    E = [[[prog.var(0.0) for _ in range(3)] for _ in range(m)] for s in range(nstages)]

    def time_op(op, s, j) -> _LinExpr:
        T_ = stages[s]["T"]
        e = _LinExpr(T_[op])
        if op == "b":
            for o in stages[s]["fwd_remat_options"]:
                e.t[fwd[s][j][o.name]] = o.time_overhead
        elif op == "w":
            for o in stages[s]["bwd_remat_options"]:
                e.t[bwd[s][j][o.name]] = o.time_overhead
        return e

    def mem_kept(op, s, j) -> _LinExpr:
        M_ = stages[s]["M"]
        e = _LinExpr(M_[op])
        if op == "f":
            for o in stages[s]["fwd_remat_options"]:
                e.t[fwd[s][j][o.name]] = -o.mem_freed
        elif op == "b":
            for o in stages[s]["bwd_remat_options"]:
                e.t[bwd[s][j][o.name]] = -o.mem_freed
        return e

    def delta_mem(op, s, j) -> _LinExpr:
        if op == "f":
            return mem_kept("f", s, j)
        prev = "f" if op == "b" else "b"
        return mem_kept(op, s, j).add(mem_kept(prev, s, j), -1.0)

    def peak_mem(op, s, j) -> _LinExpr:
        pk = stages[s]["Mpeak"]
        pF, pB, pW, pNG = pk["f"], pk["b"], pk["w"], pk["f_no_grad"]
        mf, mb_ = stages[s]["M"]["f"], stages[s]["M"]["b"]
        if op == "f":
            e = _LinExpr(pF)
            e.t[fwd[s][j]["full_fwd"]] = pNG - pF
            return e
        if op == "b":
            e = _LinExpr(pB)
            e.t[fwd[s][j]["full_fwd"]] = max(pF, mf + pB) - pB
            if "offload" in fwd[s][j]:
                e.t[fwd[s][j]["offload"]] = stages[s]["act"]  # prefetched copy is live during B
            return e
        e = _LinExpr(pW)
        e.t[bwd[s][j]["full_bwd"]] = max(pF, mf + pB, mb_ + pW) - pW
        e.t[bwd[s][j]["activations_bwd"]] = pNG - pW
        return e

    Tmax = prog.var(max(sum(sum(stages[s]["T"][o] for o in "fbw") * m for s in on_rank[i]) for i in range(p)))
    for i in range(p):
        if not sched[i]:
            continue
        fo, fs, fj = sched[i][0]
        lo_, ls, lj = sched[i][-1]
        span = _LinExpr(0.0, {E[ls][lj][_OP_INDEX[lo_]]: 1.0}).add(_LinExpr(0.0, {E[fs][fj][_OP_INDEX[fo]]: 1.0}), -1.0).add(time_op(fo, fs, fj))
        span.t[Tmax] = span.t.get(Tmax, 0.0) - 1.0
        prog.leq(span, 0.0)
    first = _LinExpr(0.0, {E[0][0][0]: 1.0}).add(time_op("f", 0, 0), -1.0)
    prog.eq(first, 0.0)

    for i in range(p):
        kept = _LinExpr(2.0 * sum(stages[s]["Mparams"] for s in on_rank[i]))  # weights + gradients
        for k, (op, s, j) in enumerate(sched[i]):
            idx = _OP_INDEX[op]
            me = _LinExpr(0.0, {E[s][j][idx]: 1.0})
            if op == "f" and s != 0:
                tc = stages[s - 1]["Tcomm"] if plc[s - 1] != plc[s] else 0.0
                prog.geq(me.copy().add(_LinExpr(tc, {E[s - 1][j][idx]: 1.0}), -1.0).add(time_op(op, s, j), -1.0), 0.0)
            elif op == "b" and s != nstages - 1:
                tc = stages[s]["Tcomm"] if plc[s + 1] != plc[s] else 0.0
                prog.geq(me.copy().add(_LinExpr(tc, {E[s + 1][j][idx]: 1.0}), -1.0).add(time_op(op, s, j), -1.0), 0.0)
            elif op == "b":
                prog.geq(me.copy().add(_LinExpr(0.0, {E[s][j][0]: 1.0}), -1.0).add(time_op(op, s, j), -1.0), 0.0)
            if op == "w":
                prog.geq(me.copy().add(_LinExpr(0.0, {E[s][j][1]: 1.0}), -1.0).add(time_op(op, s, j), -1.0), 0.0)
            if k:
                po, ps, pj = sched[i][k - 1]
                prog.geq(me.copy().add(_LinExpr(0.0, {E[ps][pj][_OP_INDEX[po]]: 1.0}), -1.0).add(time_op(op, s, j), -1.0), 0.0)
            prog.leq(kept.copy().add(peak_mem(op, s, j)), MGpu)
            kept.add(delta_mem(op, s, j))
        if offload:
            copy = _LinExpr(0.0)
            for s in on_rank[i]:
                ms_both_ways = 2.0 * stages[s]["act"] / 1024.0 / prm["pcie_gbs"] * 1e3
                for j in range(m):
                    copy.t[fwd[s][j]["offload"]] = ms_both_ways
            copy.t[Tmax] = -1.0
            prog.leq(copy, 0.0)  # PCIe cannot move more than fits in the step

    for s in range(nstages):
        for j in range(m):
            prog.leq(_LinExpr(0.0, {v: 1.0 for v in fwd[s][j].values()}), 1.0)
            prog.leq(_LinExpr(0.0, {v: 1.0 for v in bwd[s][j].values()}), 1.0)

    t0 = time.time()
    res = prog.solve(_LinExpr(0.0, {Tmax: 1.0}), time_limit, gap_rel_limit)
    took = time.time() - t0
    if res.x is None:
        if res.status in (2,) or "infeasible" in str(res.message).lower():
            raise RuntimeError(
                f"ILP is infeasible: cannot fit the schedule within {memory_budget} MB. "
                "Try increasing memory_budget, reducing n_micro_batches or using a different scheduler."
            )
        raise RuntimeError(f"ILP solver returned no solution within {time_limit}s: {res.message}")
    x = res.x
    solution = {"placement": list(plc), "objective": float(x[Tmax]), "order": [op for rank_ops in sched for op in rank_ops]}
    names = ["full_fwd", "activations_bwd", "full_bwd"] + (["offload"] if offload else [])
    for name in names:
        table = fwd if name in ("full_fwd", "offload") else bwd
        solution[name] = [[int(round(x[table[s][j][name]])) for j in range(m)] for s in range(nstages)]
    peaks = []
    for i in range(p):
        acc = 2.0 * sum(stages[s]["Mparams"] for s in on_rank[i])
        pk = acc
        for op, s, j in sched[i]:
            pk = max(pk, acc + peak_mem(op, s, j).value(x))
            acc += delta_mem(op, s, j).value(x)
        peaks.append(pk)
    solution["peak_mems"] = peaks
    logger.info("ILP solved in %.2fs: objective=%.1fms, peak_mems=%s", took, solution["objective"], [f"{v:.0f}MB" for v in peaks])
    return solution


# =======================================================================================
# 3. applying a solution
# =======================================================================================


def _whole_stage(name, _module=None) -> bool:
    return name == ""


class RematScheduler:
    """``base`` schedule + the decisions of a ``solve_remat`` solution.

    ``full_fwd``         F gets ``REMAT_STRATEGY`` = checkpoint the whole stage
    ``activations_bwd``  B gets ``RECOMPUTE_ACTIVATIONS``; a ``RECOMPUTE_FORWARD`` is placed right
                         before the W of the same (stage, micro-batch)
    ``full_bwd``         additionally ``RECOMPUTE_GRADIENTS`` on B, ``SAVE`` on the recompute-forward
                         and a ``RECOMPUTE_BACKWARD_INPUTS`` before the W
    ``offload``          F and B get ``ACTIVATION_OFFLOAD`` and a ``PREFETCH_ACTIVATIONS`` precedes B
    """

    def __init__(self, base_scheduler, solution: dict, prefetching_time: int = 1):
        self.base_scheduler = base_scheduler
        self.solution = solution
        self.prefetching_time = prefetching_time

    @property
    def makespan(self) -> float:
        return self.solution["objective"]

    def _chosen(self, name: str, op: Operation) -> bool:
        table = self.solution.get(name) or []
        try:
            return bool(table[op.block_id][op.mb_id])
        except IndexError:
            return False

    def __call__(self, placement, nmb) -> List[Operation]:
        schedule = self.base_scheduler(placement, nmb)
        before_w: Dict[Tuple[int, int], List[Operation]] = {}
        for op in schedule:
            if op.op is T.FORWARD and self._chosen("full_fwd", op):
                op.options[OpOptions.REMAT_STRATEGY] = _whole_stage
            elif op.op is T.BACKWARD_INPUTS:
                acts, full = self._chosen("activations_bwd", op), self._chosen("full_bwd", op)
                if not (acts or full):
                    continue
                op.options[OpOptions.RECOMPUTE_ACTIVATIONS] = True
                rf = Operation(op.block_id, op.mb_id, T.RECOMPUTE_FORWARD, op.rank)
                extra = [rf]
                if full:
                    rf.options[OpOptions.SAVE] = True
                    op.options[OpOptions.RECOMPUTE_GRADIENTS] = True
                    extra.append(Operation(op.block_id, op.mb_id, T.RECOMPUTE_BACKWARD_INPUTS, op.rank))
                before_w[(op.block_id, op.mb_id)] = extra
        out: List[Operation] = []
        for op in schedule:
            if op.op is T.BACKWARD_PARAMS:
                out.extend(before_w.pop((op.block_id, op.mb_id), ()))
            out.append(op)
        off = self.solution.get("offload")
        if off:
            chosen = {(s, j) for s, row in enumerate(off) for j, v in enumerate(row) if v}
            if chosen:
                out = apply_offload(out, chosen, self.prefetching_time)
        return out


def _rank_and_bcast(worker: int, group):
    """(my global rank, broadcast function) for solution hand-off; identity without dist."""
    if dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1:
        def bcast(obj_list):
            dist.broadcast_object_list(obj_list, src=worker)
            return obj_list
        return dist.get_rank(), bcast
    return worker, (lambda obj_list: obj_list)


def stagerematify(scheduler, stats: List[dict], budget: float, worker: int = 0, group=None, offload: bool = False, **solver_kwargs):
    """Scheduler that solves the ILP for ``scheduler`` on rank ``worker`` the first time it
    is called for a given number of micro-batches and applies the solution everywhere."""
    base = resolve(scheduler, SCHEDULERS)

    def StageRemat(placement, nmb) -> List[Operation]:
        me, bcast = _rank_and_bcast(worker, group)
        box = [None]
        if me == worker:
            try:
                box[0] = solve_remat(stats, placement, base, nmb, budget, offload=offload, **solver_kwargs)
            except RuntimeError as exc:
                box[0] = exc
        box = bcast(box)
        if isinstance(box[0], Exception):
            raise box[0]
        StageRemat.solution = box[0]
        return RematScheduler(base, box[0])(placement, nmb)

    StageRemat.solution = None
    return StageRemat


class AutoScheduler:
    """Solve the remat ILP for every registered base schedule and keep the smallest
    makespan.  Schedules whose placement requirements do not match simply fail and are
    skipped.  The other ranks wait on one broadcast per candidate, which doubles as a
    keep-alive for process-group watchdogs during long solves."""

    EXCLUDED = ("auto", "fixed", "full_remat", "inference")

    def __init__(self, stats: List[dict], budget: float, worker: int = 0, group=None, offload: bool = False, **solver_kwargs):
        self.stats, self.budget, self.worker, self.group = stats, budget, worker, group
        self.offload, self.solver_kwargs = offload, solver_kwargs
        self.schedulers = [k for k in SCHEDULERS.available() if k not in self.EXCLUDED]
        self.best: Optional[Tuple[float, str, dict]] = None

    def __call__(self, placement, nmb) -> List[Operation]:
        me, bcast = _rank_and_bcast(self.worker, self.group)
        best = (float("inf"), None, None)
        for name in self.schedulers:
            note = [("keepalive", name)]
            if me == self.worker:
                try:
                    sol = solve_remat(self.stats, placement, SCHEDULERS[name], nmb, self.budget, offload=self.offload, **self.solver_kwargs)
                    if sol["objective"] < best[0]:
                        best = (sol["objective"], name, sol)
                except Exception as exc:  # wrong placement shape for this schedule, infeasible budget, ...
                    logger.info("ILP for scheduler %s skipped: %s", name, exc)
            bcast(note)
        box = bcast([best])
        objective, name, solution = box[0]
        if name is None:
            raise RuntimeError(f"no schedule fits within {self.budget} MB on placement {list(placement)}")
        logger.info("Best scheduler: %s with %.2fms makespan", name, objective)
        self.best = box[0]
        return RematScheduler(SCHEDULERS[name], solution)(placement, nmb)
