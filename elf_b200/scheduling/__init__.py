"""Schedule IR, the static schedule zoo, comm scheduling, simulation and ILP remat."""

from .scheduling import *  # noqa: F401,F403
from .scheduling import schedule_to_str, check_schedule_validity, OpOptions, Operation, OperationType
from .comm_scheduling import *  # noqa: F401,F403
from .schedulers import *  # noqa: F401,F403
from .simulator import simulate, replay_comms, DeadlockError, SimResult

from ..registry import SCHEDULERS, COMM_SCHEDULERS


def _auto_placeholder(*_args, **_kwargs):
    raise RuntimeError(
        "scheduler='auto' picks the best schedule under a memory budget: pass memory_budget=<MB> to "
        "Pipeline, or name a scheduler (" + ", ".join(k for k in SCHEDULERS.available() if k != "auto") + ")"
    )


SCHEDULERS.register(["afab", "gpipe"], generate_afab_schedule, "All Forward All Backward as in GPipe https://arxiv.org/abs/1811.06965")
SCHEDULERS.register(["1f1b", "megatron"], generate_1f1b_schedule, "One Forward One Backward (PipeDream-flush https://arxiv.org/abs/1806.03377); interleaved when several stages share a rank")
SCHEDULERS.register("hanayo", generate_hanayo_schedule, "Hanayo wave schedule https://dl.acm.org/doi/10.1145/3581784.3607073")
SCHEDULERS.register("full_remat", generate_full_remat_schedule, "GPipe with every stage checkpointed, last rank keeps activations")
SCHEDULERS.register("zbh1", generate_zbh1_schedule, "ZB-H1 https://arxiv.org/abs/2401.10241 (1F1B memory)")
SCHEDULERS.register("zbh2", generate_zbh2_schedule, "ZB-H2 https://arxiv.org/abs/2401.10241 (zero bubble, 2x memory)")
SCHEDULERS.register("zbv", generate_zbv_schedule, "ZB-V https://arxiv.org/abs/2401.10241 on a V placement, any number of micro-batches")
SCHEDULERS.register("inference", generate_inference_schedule, "Forward passes only")
SCHEDULERS.register("fixed", FixedSchedule, "Replay a {'order': [(f|b|w, block, mb), ...]} dictionary")
SCHEDULERS.register("auto", _auto_placeholder, "Solve the remat ILP for every base schedule and keep the fastest (needs memory_budget)")

COMM_SCHEDULERS.register("topo", topological_sort, "Plain topological order; each send next to its recv")
COMM_SCHEDULERS.register("simulation", smart_topological_sort, "Lock-step simulation; all ready transfers happen together each round")
COMM_SCHEDULERS.register("pipelined", pipelined_topological_sort, "recv posted before, send issued after each compute op, for comm/compute overlap")

__all__ = [
    "schedule_to_str",
    "check_schedule_validity",
    "add_comms",
    "OpOptions",
    "Operation",
    "OperationType",
    "simulate",
    "replay_comms",
]
