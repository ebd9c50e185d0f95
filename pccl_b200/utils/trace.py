"""Reading the engine's device timeline.

``Engine.set_trace(True)`` (or ``PCCL_TRACE=1``) makes the plan interpreter stamp
``%globaltimer`` four times per step; ``Engine.trace(name)`` returns the stamps of the most
recent launch.  The functions here turn that list into per-phase figures: how long each kind of
step moved data, at what rate per NVLink direction, and how long chains sat in barriers or
waits in between.  It stands where the reference uses an external timeline profiler
(tests/prof_nvtx.py:1-101 runs the workload under nsys, tests/parse_nsys.py:18-143 reads the
exported tables); here the kernel reports its own timeline, so no profiler is needed.
"""

from __future__ import annotations

from collections import defaultdict
from typing import Any, Dict, Iterable, List

#: bytes that cross this GPU's NVLink per payload byte of a step, as (outbound, inbound) factors of
#: the world size W.  A pull copy only receives; an in-switch reduction sends this rank's copy of
#: every slice some rank reduces (W slices in total while all ranks run the step) and receives its
#: own slice; an in-switch broadcast sends one slice and receives W.
_LINK_FACTORS = {
    "copy": lambda w: (1.0, 1.0),
    "put": lambda w: (1.0, 1.0),
    "reduce": lambda w: (1.0, 1.0),
    "reduce_multi": lambda w: (w - 1.0, w - 1.0),
    "multimem.reduce": lambda w: (float(w), 1.0),
    "multimem.store": lambda w: (1.0, float(w)),
    "multimem.allreduce": lambda w: (w + 1.0, w + 1.0),
}


def phases(trace: Iterable[Dict[str, Any]], world: int) -> List[Dict[str, Any]]:
    """One row per step kind: steps, payload bytes, the span from the first start to the last end
    of that kind, the mean duration of one step, and GB/s per NVLink direction over the span."""
    rows: Dict[str, Dict[str, Any]] = {}
    for step in trace:
        kind = step["kind"]
        if kind == "noop" or not step["bytes"]:
            continue
        row = rows.setdefault(kind, {"kind": kind, "steps": 0, "bytes": 0, "first_ns": None, "last_ns": 0,
                                     "busy_ns": 0})
        row["steps"] += 1
        row["bytes"] += step["bytes"]
        begin, end = step["t_data_ns"], step["t_done_ns"]
        row["first_ns"] = begin if row["first_ns"] is None else min(row["first_ns"], begin)
        row["last_ns"] = max(row["last_ns"], end)
        row["busy_ns"] += max(0, end - begin)
    out = []
    for row in rows.values():
        span = max(1, row["last_ns"] - (row["first_ns"] or 0))
        tx, rx = _LINK_FACTORS.get(row["kind"], lambda w: (1.0, 1.0))(world)
        row["span_us"] = span / 1e3
        row["mean_step_us"] = row["busy_ns"] / row["steps"] / 1e3
        row["tx_gbs"] = row["bytes"] * tx / span
        row["rx_gbs"] = row["bytes"] * rx / span
        out.append(row)
    return sorted(out, key=lambda r: r["first_ns"] or 0)


def waits(trace: Iterable[Dict[str, Any]]) -> Dict[str, float]:
    """Microseconds per chain, averaged over chains: waiting (reached -> data start), moving data,
    and posting signals (done -> posted); plus the launch's total span."""
    per_chain = defaultdict(lambda: [0, 0, 0])
    end = 0
    for step in trace:
        acc = per_chain[step["chain"]]
        acc[0] += max(0, step["t_data_ns"] - step["t_reached_ns"])
        acc[1] += max(0, step["t_done_ns"] - step["t_data_ns"])
        acc[2] += max(0, step["t_posted_ns"] - step["t_done_ns"])
        end = max(end, step["t_posted_ns"])
    n = max(1, len(per_chain))
    return {"wait_us": sum(a[0] for a in per_chain.values()) / n / 1e3,
            "data_us": sum(a[1] for a in per_chain.values()) / n / 1e3,
            "post_us": sum(a[2] for a in per_chain.values()) / n / 1e3,
            "total_us": end / 1e3, "chains": len(per_chain)}


def summarize(trace: List[Dict[str, Any]], world: int) -> str:
    """Human-readable table of ``phases`` and ``waits``."""
    lines = [f"{'phase':<20}{'steps':>6}{'MB':>10}{'span us':>10}{'step us':>10}{'tx GB/s':>10}{'rx GB/s':>10}"]
    for row in phases(trace, world):
        lines.append(f"{row['kind']:<20}{row['steps']:>6}{row['bytes'] / 1e6:>10.1f}{row['span_us']:>10.1f}"
                     f"{row['mean_step_us']:>10.1f}{row['tx_gbs']:>10.1f}{row['rx_gbs']:>10.1f}")
    w = waits(trace)
    lines.append(f"per chain ({w['chains']} chains): waiting {w['wait_us']:.1f} us, moving {w['data_us']:.1f} us, "
                 f"posting {w['post_us']:.1f} us; launch span {w['total_us']:.1f} us")
    return "\n".join(lines)
