"""Kernel-time breakdown and compute / communication overlap of a ``torch.profiler`` chrome trace.

``parse_trace_file(path)`` reads the JSON (optionally gzipped), keeps the GPU kernel events, classifies them
as communication (NCCL, this package's peer-memory collectives, copy-engine peer copies) or compute, and
reports per-kernel totals, the busy time of each class, how much of the communication time is hidden under
compute kernels and how much is exposed, per step when ``ProfilerStep#`` annotations are present.
(Reference: atorch/utils/parse_trace_json.py:20-330, which needs pandas; this one is plain Python.)
"""
from __future__ import annotations

import argparse
import gzip
import json
from collections import defaultdict
from typing import Dict, List, Tuple

COMM_HINTS = ("nccl", "p2p_", "allreduce", "all_reduce", "allgather", "all_gather", "reduce_scatter", "moe_scatter",
              "moe_gather", "pad_wait", "pad_signal", "Memcpy PtoP", "Memcpy DtoD (Device -> Device) peer")


def is_comm(name: str) -> bool:
    low = name.lower()
    return any(h.lower() in low for h in COMM_HINTS)


def _merge(intervals: List[Tuple[float, float]]) -> List[Tuple[float, float]]:
    out: List[Tuple[float, float]] = []
    for s, e in sorted(intervals):
        if out and s <= out[-1][1]:
            out[-1] = (out[-1][0], max(out[-1][1], e))
        else:
            out.append((s, e))
    return out


def _length(iv: List[Tuple[float, float]]) -> float:
    return sum(e - s for s, e in iv)


def _intersect(a: List[Tuple[float, float]], b: List[Tuple[float, float]]) -> float:
    i = j = 0
    tot = 0.0
    while i < len(a) and j < len(b):
        s, e = max(a[i][0], b[j][0]), min(a[i][1], b[j][1])
        if e > s:
            tot += e - s
        if a[i][1] < b[j][1]:
            i += 1
        else:
            j += 1
    return tot


def load_events(path: str) -> List[dict]:
    opener = gzip.open if path.endswith(".gz") else open
    with opener(path, "rt") as f:
        obj = json.load(f)
    return obj["traceEvents"] if isinstance(obj, dict) else obj


def analyze(events: List[dict]) -> Dict:
    kernels = [e for e in events if e.get("ph") == "X" and e.get("cat") in ("kernel", "gpu_memcpy", "gpu_memset")]
    per_kernel = defaultdict(lambda: [0, 0.0])
    comp, comm = [], []
    for e in kernels:
        name, ts, dur = e.get("name", ""), float(e["ts"]), float(e.get("dur", 0.0))
        per_kernel[name][0] += 1
        per_kernel[name][1] += dur
        (comm if is_comm(name) else comp).append((ts, ts + dur))
    comp_m, comm_m = _merge(comp), _merge(comm)
    hidden = _intersect(comp_m, comm_m)
    # mean duration of each compute kernel with and without a communication kernel or peer copy in flight
    contention = defaultdict(lambda: [0, 0.0, 0, 0.0])
    starts = [s for s, _ in comm_m]
    import bisect
    for e in kernels:
        name, ts, dur = e.get("name", ""), float(e["ts"]), float(e.get("dur", 0.0))
        if is_comm(name):
            continue
        k = bisect.bisect_right(starts, ts + dur) - 1
        busy = k >= 0 and comm_m[k][1] > ts
        c = contention[name]
        c[2 if busy else 0] += 1
        c[3 if busy else 1] += dur
    steps = [e for e in events if e.get("ph") == "X" and str(e.get("name", "")).startswith("ProfilerStep#")]
    span = (max(e for _, e in comp_m + comm_m) - min(s for s, _ in comp_m + comm_m)) if (comp_m or comm_m) else 0.0
    return {
        "n_kernels": len(kernels), "n_steps": len(steps), "span_us": span,
        "compute_busy_us": _length(comp_m), "comm_busy_us": _length(comm_m),
        "comm_hidden_us": hidden, "comm_exposed_us": _length(comm_m) - hidden,
        "overlap_ratio": hidden / _length(comm_m) if comm_m else 1.0,
        "idle_us": max(span - _length(_merge(comp + comm)), 0.0),
        "contention": {n: c for n, c in contention.items()},
        "top_kernels": sorted(((n, c, d) for n, (c, d) in per_kernel.items()), key=lambda t: -t[2])[:25],
    }


def parse_trace_file(json_file: str, verbose: bool = False) -> Dict:
    res = analyze(load_events(json_file))
    if verbose:
        print_profiler_summary(res)
    return res


def print_profiler_summary(res: Dict, all_summary_path=None) -> None:
    n = max(res["n_steps"], 1)
    lines = [f"kernels {res['n_kernels']}  steps {res['n_steps']}  span {res['span_us'] / 1e3:.2f} ms",
             f"per step: compute {res['compute_busy_us'] / n / 1e3:.2f} ms, communication {res['comm_busy_us'] / n / 1e3:.2f} ms "
             f"(hidden {res['comm_hidden_us'] / n / 1e3:.2f}, exposed {res['comm_exposed_us'] / n / 1e3:.2f}), "
             f"idle {res['idle_us'] / n / 1e3:.2f} ms, overlap {100 * res['overlap_ratio']:.1f} %"]
    for name, cnt, dur in res["top_kernels"]:
        line = f"{dur / n / 1e3:9.3f} ms/step x{cnt // n:5d}  {name[:110]}"
        c = res.get("contention", {}).get(name)
        if c and c[0] and c[2]:
            line += f"  [alone {c[1] / c[0]:.1f} us x{c[0]}, with communication in flight {c[3] / c[2]:.1f} us x{c[2]}]"
        lines.append(line)
    text = "\n".join(lines)
    print(text)
    if all_summary_path:
        with open(all_summary_path, "w") as f:
            f.write(text + "\n")


def main(argv=None) -> None:
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("trace")
    ap.add_argument("--out", default=None)
    ap.add_argument("--steps", type=int, default=0, help="number of training steps in the trace when it carries "
                                                         "no ProfilerStep annotations")
    a = ap.parse_args(argv)
    res = parse_trace_file(a.trace)
    if a.steps > 0:
        res["n_steps"] = a.steps
    print_profiler_summary(res, a.out)


if __name__ == "__main__":
    main()
