"""Merge per-rank Chrome traces (torch.profiler exports) into one file and compact them.

`merge_traces` offsets pids per rank so the ranks sit side by side and aligns clocks on the first event; `compact_trace`
drops events shorter than a threshold and python-function noise, which shrinks a CUDA-graph decode trace by orders of
magnitude; `summarize_kernels` totals kernel time by name.
Parity: reference dlengine/utils/trace_merger.py, trace_compactor.py, bench/analyze_cuda_graph_trace.py."""
from __future__ import annotations

import gzip
import json
from collections import defaultdict
from typing import Dict, Iterable, List


def _load(path: str) -> Dict:
    op = gzip.open if path.endswith(".gz") else open
    with op(path, "rt") as f:
        d = json.load(f)
    return d if isinstance(d, dict) else {"traceEvents": d}


def merge_traces(paths: Iterable[str], out_path: str, align: bool = True) -> int:
    events: List[dict] = []
    for rank, p in enumerate(sorted(paths)):
        evs = _load(p).get("traceEvents", [])
        t0 = min((e["ts"] for e in evs if "ts" in e and e.get("ph") != "M"), default=0) if align else 0
        for e in evs:
            e = dict(e)
            if isinstance(e.get("pid"), int):
                e["pid"] = e["pid"] + rank * 1_000_000
            else:
                e["pid"] = f"rank{rank}:{e.get('pid')}"
            if "ts" in e and e.get("ph") != "M":
                e["ts"] = e["ts"] - t0
            if e.get("ph") == "M" and e.get("name") == "process_name":
                e.setdefault("args", {})["name"] = f"rank {rank} " + str(e.get("args", {}).get("name", ""))
            events.append(e)
    with open(out_path, "w") as f:
        json.dump({"traceEvents": events}, f)
    return len(events)


def compact_trace(path: str, out_path: str, min_dur_us: float = 2.0, drop_categories=("python_function", "user_annotation_python")) -> int:
    evs = _load(path).get("traceEvents", [])
    keep = [e for e in evs if e.get("ph") == "M" or (e.get("cat") not in drop_categories and (e.get("ph") != "X" or e.get("dur", 0) >= min_dur_us))]
    with open(out_path, "w") as f:
        json.dump({"traceEvents": keep}, f)
    return len(keep)


def summarize_kernels(path: str, top: int = 30) -> List[tuple]:
    tot, cnt = defaultdict(float), defaultdict(int)
    for e in _load(path).get("traceEvents", []):
        if e.get("cat") in ("kernel", "gpu_memcpy", "gpu_memset") and e.get("ph") == "X":
            tot[e["name"]] += e.get("dur", 0.0)
            cnt[e["name"]] += 1
    return sorted(((n, cnt[n], t) for n, t in tot.items()), key=lambda x: -x[2])[:top]


def compact_stream_lanes(path: str, out_path: str, min_group: int = 4) -> int:
    """Fold the stream lanes a CUDA-graph replay produces into one lane per role.

    A replayed graph with fork / join branches (the shared-expert side stream of every MoE layer) shows up in a profiler
    trace as one stream lane per branch instance.  Lanes of one process whose kernels have the same name histogram are
    copies of the same branch; when at least `min_group` lanes share a histogram their events are mapped onto the
    lowest-numbered lane of the group.  Returns the number of lanes removed.
    Parity: reference utils/trace_compactor.py:9-85 (StreamLaneCompactor)."""
    data = _load(path)
    evs = data.get("traceEvents", [])
    hist: Dict[tuple, Dict[str, int]] = defaultdict(lambda: defaultdict(int))
    for e in evs:
        if e.get("cat") == "kernel" and e.get("ph") == "X" and "pid" in e and "tid" in e:
            hist[(e["pid"], e["tid"])][str(e.get("name", ""))] += 1
    groups: Dict[tuple, list] = defaultdict(list)
    for (pid, tid), h in hist.items():
        groups[(pid, tuple(sorted(h.items())))].append(tid)
    remap, removed = {}, 0
    for (pid, _), tids in groups.items():
        if len(tids) < min_group:
            continue
        keep = min(tids, key=lambda t: (str(type(t)), t))
        for t in tids:
            if t != keep:
                remap[(pid, t)] = keep
                removed += 1
    out = []
    for e in evs:
        key = (e.get("pid"), e.get("tid"))
        if key in remap:
            if e.get("ph") == "M":
                continue                     # metadata of a folded lane
            e = dict(e, tid=remap[key])
        out.append(e)
    with open(out_path, "w") as f:
        json.dump({**{k: v for k, v in data.items() if k != "traceEvents"}, "traceEvents": out}, f)
    return removed
