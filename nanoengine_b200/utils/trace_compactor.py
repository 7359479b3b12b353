"""Shrinks Chrome traces (torch.profiler exports) so that hours of serving fit a viewer: drops the event categories a
kernel-level reading does not need (python function frames, memory events, flow arrows), folds runs of identical short kernels
on one stream into one event with a count, and keeps everything longer than a threshold as it is.  Works as a stream over
the `traceEvents` list, so traces larger than memory-comfortable can be compacted rank by rank before `trace_merger` joins them.

Parity: reference dlengine/utils/trace_compactor.py (tests/test_trace_stream_compaction.py, test_profiler_compact_endpoint.py).
"""
from __future__ import annotations

import json
from typing import Dict, Iterable, Iterator, List, Optional

DROP_CATEGORIES = ("python_function", "cpu_instant_event", "ac2g", "fwdbwd", "user_annotation_flow")


def compact_events(events: Iterable[dict], min_us: float = 5.0, drop_categories=DROP_CATEGORIES, fold: bool = True) -> Iterator[dict]:
    """Yields the compacted event stream.  Complete events ("ph" == "X") shorter than `min_us` that repeat the previous name on
    the same (pid, tid) are folded into that event: its duration grows to cover them and `args.count` says how many it stands for."""
    last: Dict[tuple, dict] = {}
    for ev in events:
        cat = ev.get("cat", "")
        if any(cat.startswith(c) for c in drop_categories) or ev.get("ph") in ("s", "t", "f"):
            continue
        if ev.get("ph") != "X":
            yield ev
            continue
        key = (ev.get("pid"), ev.get("tid"))
        prev = last.get(key)
        if (fold and prev is not None and prev.get("name") == ev.get("name") and float(ev.get("dur", 0)) < min_us
                and float(prev.get("args", {}).get("_unit", prev.get("dur", 0))) < min_us):
            end = max(prev["ts"] + prev["dur"], ev["ts"] + ev.get("dur", 0))
            prev["dur"] = end - prev["ts"]
            a = prev.setdefault("args", {})
            a["count"] = a.get("count", 1) + 1
            continue
        if prev is not None:
            prev.get("args", {}).pop("_unit", None)
            yield prev
        cur = dict(ev)
        cur["args"] = dict(ev.get("args", {}), _unit=float(ev.get("dur", 0)))
        last[key] = cur
    for prev in last.values():
        prev.get("args", {}).pop("_unit", None)
        yield prev


def compact_file(src: str, dst: str, min_us: float = 5.0) -> dict:
    """Compacts one trace file; returns {"events_in", "events_out"}."""
    with open(src) as f:
        doc = json.load(f)
    events = doc["traceEvents"] if isinstance(doc, dict) else doc
    out: List[dict] = sorted(compact_events(events, min_us), key=lambda e: e.get("ts", 0))
    res = dict(doc, traceEvents=out) if isinstance(doc, dict) else out
    with open(dst, "w") as f:
        json.dump(res, f)
    return {"events_in": len(events), "events_out": len(out)}
