#!/usr/bin/env python
"""Read a per-operation timeline written by ``bench.py --timeline FILE`` and say where every
rank of the pipeline spends the time in which it computes nothing.

For each rank: busy time, idle time split into *fill* (before its first operation), *drain*
(after its last), *waiting for a peer* (gap in front of a forward / backward-inputs operation
whose input comes from another rank) and *other gaps* (between operations that depend on
nothing remote: launch gaps, allocator, host).  Then the same operations, with their measured
durations and the order each rank really ran them in, are replayed by the timeline simulator
(``elf_b200.scheduling.simulator``) with a given hop latency, which shows how much of the
measured step the data-flow model explains.

    python benchmarks/pipeline_timeline.py timeline.json [--hop-ms 0.15] [--chrome-trace trace.json]
"""

from __future__ import annotations

import argparse
import json
import os
import re
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

_NAME = re.compile(r"(forward|backward_inputs|backward_params|recompute_forward|recompute_backward_inputs|backward)\((\d+):(\d+)\)$")


def load(path):
    with open(path) as f:
        data = json.load(f)
    placement = data["placement"]
    ranks = {}
    for r, entry in data["ranks"].items():
        ops = []
        for name, (t0, t1) in entry["timeline"].items():
            m = _NAME.match(name)
            if m:
                ops.append((t0 * 1e3, t1 * 1e3, m.group(1), int(m.group(2)), int(m.group(3))))
            else:
                ops.append((t0 * 1e3, t1 * 1e3, name, -1, -1))
        ops.sort()
        ranks[int(r)] = {"ops": ops, "total_ms": (entry.get("total_s") or 0.0) * 1e3, "host": entry.get("host_enqueue", {})}
    return placement, data.get("nmb"), ranks


def analyse(placement, ranks):
    n_stages = len(placement)
    rows = []
    step_end = max(op[1] for info in ranks.values() for op in info["ops"])
    for r in sorted(ranks):
        ops = ranks[r]["ops"]
        busy = sum(t1 - t0 for t0, t1, *_ in ops)
        fill = ops[0][0]
        drain = step_end - ops[-1][1]
        wait_peer = other = 0.0
        worst = []
        for prev, cur in zip(ops, ops[1:]):
            gap = cur[0] - prev[1]
            if gap <= 0:
                continue
            kind, stage = cur[2], cur[3]
            remote = (kind == "forward" and stage > 0 and placement[stage - 1] != r) or (
                kind == "backward_inputs" and stage < n_stages - 1 and placement[stage + 1] != r
            )
            if remote:
                wait_peer += gap
            else:
                other += gap
            worst.append((gap, f"{kind}({stage}:{cur[4]})", "peer" if remote else "local"))
        worst.sort(reverse=True)
        rows.append({"rank": r, "busy": busy, "fill": fill, "drain": drain, "wait_peer": wait_peer, "other": other, "n_ops": len(ops), "worst": worst[:5]})
    return step_end, rows


def replay(placement, nmb, ranks, hop_ms):
    """Simulated makespan for the measured durations and the measured per-rank order."""
    from elf_b200.scheduling.scheduling import Operation, OperationType as T
    from elf_b200.scheduling.simulator import simulate

    kinds = {"forward": T.FORWARD, "backward_inputs": T.BACKWARD_INPUTS, "backward_params": T.BACKWARD_PARAMS}
    sched, dur = [], {}
    extra = {r: 0.0 for r in ranks}  # loss operations: charged to the next operation of the rank
    for r in sorted(ranks):
        carry = 0.0
        for t0, t1, kind, stage, mb in ranks[r]["ops"]:
            if kind not in kinds:
                carry += t1 - t0
                continue
            op = Operation(stage, mb, kinds[kind], r)
            sched.append(op)
            dur[(stage, mb, kinds[kind])] = (t1 - t0) + carry
            carry = 0.0
    res = simulate(sched, placement, lambda op: dur.get((op.block_id, op.mb_id, op.op), 0.0), hop=hop_ms)
    return res


def chrome_trace(path_in: str, path_out: str) -> int:
    """Write every timed operation of every rank as a complete event of the Trace Event format
    (one process per rank; open the file in Perfetto or ``chrome://tracing``).  Returns the
    number of events."""
    with open(path_in) as f:
        data = json.load(f)
    colours = {"forward": "good", "backward_inputs": "bad", "backward": "terrible", "backward_params": "olive", "loss_forward": "yellow"}
    events = []
    for r, entry in sorted(data["ranks"].items(), key=lambda kv: int(kv[0])):
        events.append({"ph": "M", "pid": int(r), "name": "process_name", "args": {"name": f"rank {r}"}})
        for name, (t0, t1) in entry["timeline"].items():
            kind = name.split("(")[0].split("#")[0]
            events.append({"ph": "X", "pid": int(r), "tid": 0, "name": name.split("#")[0], "cat": kind, "ts": 1e6 * t0, "dur": 1e6 * max(0.0, t1 - t0),
                           "cname": colours.get(kind, "grey")})
    with open(path_out, "w") as f:
        json.dump({"traceEvents": events, "displayTimeUnit": "ms"}, f)
    return sum(1 for e in events if e["ph"] == "X")


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("file")
    ap.add_argument("--hop-ms", type=float, nargs="*", default=[0.0, 0.1, 0.2, 0.4])
    ap.add_argument("--chrome-trace", metavar="OUT", help="also write the operations as a Trace Event file (Perfetto / chrome://tracing)")
    args = ap.parse_args()
    if args.chrome_trace:
        print(f"wrote {chrome_trace(args.file, args.chrome_trace)} events to {args.chrome_trace}")
    placement, nmb, ranks = load(args.file)
    step_end, rows = analyse(placement, ranks)
    print(f"placement {placement}, {nmb} micro-batches; last operation ends {step_end:.1f} ms after the step's start")
    print(f"{'rank':>4} {'ops':>4} {'busy':>8} {'fill':>7} {'drain':>7} {'wait peer':>10} {'other gaps':>10}   largest gaps (ms, before op, kind)")
    for row in rows:
        worst = ", ".join(f"{g:.2f} {n} {k}" for g, n, k in row["worst"][:3])
        print(f"{row['rank']:>4} {row['n_ops']:>4} {row['busy']:>8.1f} {row['fill']:>7.1f} {row['drain']:>7.1f} {row['wait_peer']:>10.1f} {row['other']:>10.1f}   {worst}")
    mean_busy = sum(r["busy"] for r in rows) / len(rows)
    print(f"mean busy {mean_busy:.1f} ms, max busy {max(r['busy'] for r in rows):.1f} ms -> balance limit {mean_busy / max(r['busy'] for r in rows):.3f}, measured {mean_busy / step_end:.3f}")
    for hop in args.hop_ms:
        res = replay(placement, nmb, ranks, hop)
        print(f"replay with hop {hop:.2f} ms: makespan {res.makespan:.1f} ms ({100 * res.makespan / step_end:.1f} % of measured)")
    for r in sorted(ranks):
        host = ranks[r]["host"]
        if host:
            last = max(host.values()) * 1e3
            print(f"rank {r}: host issued its last compute operation {last:.1f} ms after the step's start")


if __name__ == "__main__":
    main()
