"""Turn step traces into tables: per-stream busy time, compute/communication overlap, kernel classes, top kernels.

    python -m pithtrain_b200.tools.profile.analyze workspace/profiles/qwen3 [--top 25] [--json out.json]

Input: the ``trace_rank<r>.json[.gz]`` files written by ``capture`` (Chrome trace events; GPU work is every
complete event of category ``kernel``, ``gpu_memcpy`` or ``gpu_memset`` and carries its stream id in ``args``), or
Nsight Systems exports (``nsys export --type=sqlite``; ``*.sqlite`` files, one per rank): kernels, copies and memsets
come from the ``CUPTI_ACTIVITY_KIND_*`` tables, limited to the NVTX range that ``TrainingCfg.nsys_start`` opens
(``rank=...``) when there is one, and every kernel is attributed to the engine's ``layerNN.stageK_{f,b,w}`` range that
was open on the launching thread, which gives a per-stage table as well. Per rank the tool reports

* the step window (first GPU event to last) and the time no stream was busy (launch- or host-bound gaps);
* busy time per stream (union of its intervals) — the compute stream, the communication stream, copy streams;
* for each kernel class (gemm, attention, communication, optimizer, memcpy, other) the summed duration,
  and for communication the share that ran while a compute kernel was running on another stream — the
  quantity the reference's nsys analysis calls overlap
  (.agents/skills/analyze-nsys-profile/scripts of the reference);
* the kernels with the largest total time.
"""

from __future__ import annotations

import argparse
import gzip
import json
import re
import sys
from collections import defaultdict
from pathlib import Path
from typing import Dict, Iterable, List, Tuple

GPU_CATS = {"kernel", "gpu_memcpy", "gpu_memset"}
CLASSES = [
    ("communication", re.compile(r"nccl|pt_ep_|ep_push|ep_return|ep_receive|ep_wait|ep_ack|ep_plan|ep_compact|fsdp::|symm", re.I)),
    ("attention", re.compile(r"fmha|flash|sdpa|attn|cudnn", re.I)),
    ("gemm", re.compile(r"gemm|nvjet|cutlass|cublas|xmma|tcgen05", re.I)),
    ("optimizer", re.compile(r"muon|adamw|sumsq|axpby|newton", re.I)),
]
Interval = Tuple[float, float]
STAGE_RX = re.compile(r"layer\d+\.(stage\d_[fbw])|^(prolog_[fb]|epilog_f|weight chunk|criterion|pipeline send/recv)$")


def classify(name: str, cat: str) -> str:
    if cat != "kernel":
        return "memcpy"
    for label, rx in CLASSES:
        if rx.search(name):
            return label
    return "other"


def load_events(path: Path) -> List[dict]:
    opener = gzip.open if path.suffix == ".gz" else open
    with opener(path, "rt") as f:
        data = json.load(f)
    events = data["traceEvents"] if isinstance(data, dict) else data
    out = []
    launches: Dict[int, Tuple[object, float]] = {}  # correlation id -> (thread, launch time)
    stages: Dict[object, List[Tuple[float, float, str]]] = defaultdict(list)  # thread -> (start, end, stage)
    for e in events:
        if e.get("ph") != "X" or e.get("dur") is None:
            continue
        cat, args = e.get("cat"), (e.get("args") or {})
        if cat in GPU_CATS:
            out.append({"name": e.get("name", "?"), "cat": cat, "ts": float(e["ts"]), "dur": float(e["dur"]),
                        "stream": args.get("stream", e.get("tid", 0)), "corr": args.get("correlation")})
        elif cat == "cuda_runtime" and "correlation" in args:
            launches[args["correlation"]] = ((e.get("pid"), e.get("tid")), float(e["ts"]))
        elif cat == "user_annotation":
            m = STAGE_RX.search(e.get("name", ""))
            if m:
                stages[(e.get("pid"), e.get("tid"))].append((float(e["ts"]), float(e["ts"]) + float(e["dur"]), m.group(1) or m.group(2)))
    if stages and launches:  # captured with --with-cpu: attribute every kernel to the stage range open at its launch
        import bisect

        starts = {}
        for th in stages:
            stages[th].sort()
            starts[th] = [r[0] for r in stages[th]]
        for ev in out:
            th, t = launches.get(ev.get("corr"), (None, None))
            if th in stages:
                i = bisect.bisect_right(starts[th], t) - 1
                if i >= 0 and stages[th][i][1] >= t:
                    ev["stage"] = stages[th][i][2]
    return out


def load_events_sqlite(path: Path) -> List[dict]:
    """GPU work of one Nsight Systems export as the event dicts :func:`analyze_events` takes (times in microseconds);
    events carry ``stage`` when the launch happened inside one of the engine's NVTX stage ranges."""
    import bisect
    import sqlite3

    db = sqlite3.connect(f"file:{path}?mode=ro", uri=True)
    tables = {r[0] for r in db.execute("SELECT name FROM sqlite_master WHERE type='table'")}
    strings = dict(db.execute("SELECT id, value FROM StringIds")) if "StringIds" in tables else {}
    out: List[dict] = []
    if "CUPTI_ACTIVITY_KIND_KERNEL" in tables:
        cols = {r[1] for r in db.execute("PRAGMA table_info(CUPTI_ACTIVITY_KIND_KERNEL)")}
        name_col = "demangledName" if "demangledName" in cols else "shortName"
        for start, end, stream, name_id, corr in db.execute(
                f"SELECT start, end, streamId, {name_col}, correlationId FROM CUPTI_ACTIVITY_KIND_KERNEL"):
            out.append({"name": strings.get(name_id, str(name_id)), "cat": "kernel", "ts": start / 1e3, "dur": (end - start) / 1e3,
                        "stream": stream, "corr": corr})
    for table, cat, label in (("CUPTI_ACTIVITY_KIND_MEMCPY", "gpu_memcpy", "Memcpy"), ("CUPTI_ACTIVITY_KIND_MEMSET", "gpu_memset", "Memset")):
        if table in tables:
            for start, end, stream, corr in db.execute(f"SELECT start, end, streamId, correlationId FROM {table}"):
                out.append({"name": label, "cat": cat, "ts": start / 1e3, "dur": (end - start) / 1e3, "stream": stream, "corr": corr})
    ranges = []  # (thread, start, end, text)
    if "NVTX_EVENTS" in tables:
        cols = {r[1] for r in db.execute("PRAGMA table_info(NVTX_EVENTS)")}
        text = "COALESCE(n.text, s.value)" if "textId" in cols and strings else "n.text"
        join = "LEFT JOIN StringIds s ON n.textId = s.id" if "textId" in cols and strings else ""
        for start, end, tid, txt in db.execute(f"SELECT n.start, n.end, n.globalTid, {text} FROM NVTX_EVENTS n {join} WHERE n.end IS NOT NULL"):
            if txt:
                ranges.append((tid, start, end, txt))
    window = [(s_, e_) for _, s_, e_, txt in ranges if txt.startswith("rank=")]
    if window:
        lo, hi = min(w[0] for w in window) / 1e3, max(w[1] for w in window) / 1e3
        out = [e for e in out if e["ts"] >= lo and e["ts"] + e["dur"] <= hi]
    if "CUPTI_ACTIVITY_KIND_RUNTIME" in tables and ranges:
        launch = {corr: (tid, start) for corr, tid, start in db.execute("SELECT correlationId, globalTid, start FROM CUPTI_ACTIVITY_KIND_RUNTIME")}
        per_thread: Dict[int, List[Tuple[int, int, str]]] = defaultdict(list)
        for tid, start, end, txt in ranges:
            m = STAGE_RX.search(txt)
            if m:
                per_thread[tid].append((start, end, m.group(1) or m.group(2)))
        starts = {}
        for tid in per_thread:
            per_thread[tid].sort()
            starts[tid] = [r[0] for r in per_thread[tid]]
        for e in out:
            tid, t = launch.get(e.get("corr"), (None, None))
            if tid in per_thread:
                # stage ranges of one thread do not nest: the candidate is the last one that started before the launch
                i = bisect.bisect_right(starts[tid], t) - 1
                if i >= 0 and per_thread[tid][i][1] >= t:
                    e["stage"] = per_thread[tid][i][2]
    db.close()
    return out


def union(intervals: Iterable[Interval]) -> List[Interval]:
    merged: List[Interval] = []
    for s, e in sorted(intervals):
        if merged and s <= merged[-1][1]:
            if e > merged[-1][1]:
                merged[-1] = (merged[-1][0], e)
        else:
            merged.append((s, e))
    return merged


def total(intervals: Iterable[Interval]) -> float:
    return sum(e - s for s, e in intervals)


def intersect(a: List[Interval], b: List[Interval]) -> float:
    """Summed length of the intersection of two merged interval lists."""
    i = j = 0
    acc = 0.0
    while i < len(a) and j < len(b):
        lo, hi = max(a[i][0], b[j][0]), min(a[i][1], b[j][1])
        if hi > lo:
            acc += hi - lo
        if a[i][1] < b[j][1]:
            i += 1
        else:
            j += 1
    return acc


def analyze_events(events: List[dict], top: int = 25) -> Dict:
    if not events:
        return {"window_us": 0.0, "streams": {}, "classes": {}, "top": [], "idle_us": 0.0, "comm_overlap": None}
    t0 = min(e["ts"] for e in events)
    t1 = max(e["ts"] + e["dur"] for e in events)
    by_stream: Dict[str, List[Interval]] = defaultdict(list)
    by_class: Dict[str, List[dict]] = defaultdict(list)
    by_name: Dict[str, List[float]] = defaultdict(list)
    for e in events:
        iv = (e["ts"], e["ts"] + e["dur"])
        by_stream[str(e["stream"])].append(iv)
        c = classify(e["name"], e["cat"])
        e["cls"] = c
        by_class[c].append(e)
        by_name[e["name"]].append(e["dur"])
    busy_all = union((e["ts"], e["ts"] + e["dur"]) for e in events)
    streams = {s: {"busy_us": total(union(iv)), "launches": len(iv)} for s, iv in by_stream.items()}
    comm = union((e["ts"], e["ts"] + e["dur"]) for e in by_class.get("communication", []))
    # a stream counts as a communication stream when most of its busy time is communication kernels
    # (a stray collective on the compute stream must not turn it into one)
    comm_time: Dict[str, float] = defaultdict(float)
    all_time: Dict[str, float] = defaultdict(float)
    for e in events:
        all_time[str(e["stream"])] += e["dur"]
        if e["cls"] == "communication":
            comm_time[str(e["stream"])] += e["dur"]
    comm_streams = {s for s, t in comm_time.items() if t > 0.5 * all_time[s]}
    compute = union((e["ts"], e["ts"] + e["dur"]) for e in events
                    if e["cls"] in ("gemm", "attention", "other", "optimizer") and str(e["stream"]) not in comm_streams)
    classes = {c: {"sum_us": sum(e["dur"] for e in evs), "launches": len(evs)} for c, evs in by_class.items()}
    overlap = (intersect(comm, compute) / total(comm)) if comm and total(comm) > 0 else None
    ranked = sorted(by_name.items(), key=lambda kv: -sum(kv[1]))[:top]
    stages: Dict[str, Dict[str, float]] = {}
    for e in events:
        st = e.get("stage")
        if st is None:
            continue
        row = stages.setdefault(st, {"sum_us": 0.0, "launches": 0, "comm_us": 0.0})
        row["sum_us"] += e["dur"]
        row["launches"] += 1
        if e["cls"] == "communication":
            row["comm_us"] += e["dur"]
    for st, row in stages.items():
        mine = union((e["ts"], e["ts"] + e["dur"]) for e in events if e.get("stage") == st and e["cls"] == "communication")
        row["comm_overlap"] = (intersect(mine, compute) / total(mine)) if mine and total(mine) > 0 else None
    return {"stages": stages, "window_us": t1 - t0, "idle_us": (t1 - t0) - total(busy_all), "streams": streams, "classes": classes,
            "comm_overlap": overlap, "comm_exposed_us": (total(comm) - intersect(comm, compute)) if comm else 0.0,
            "top": [{"name": n, "sum_us": sum(d), "launches": len(d), "mean_us": sum(d) / len(d)} for n, d in ranked]}


def render(rank: str, r: Dict) -> List[str]:
    w = r["window_us"] or 1.0
    out = [f"== {rank}: step window {w / 1e3:.2f} ms, all streams idle {r['idle_us'] / 1e3:.2f} ms ({100 * r['idle_us'] / w:.1f}%)"]
    out.append("  stream            busy ms   share  launches")
    for s, v in sorted(r["streams"].items(), key=lambda kv: -kv[1]["busy_us"]):
        out.append(f"  {s:<14s}{v['busy_us'] / 1e3:11.2f}{100 * v['busy_us'] / w:7.1f}%{v['launches']:10d}")
    out.append("  class              sum ms   share  launches")
    for c, v in sorted(r["classes"].items(), key=lambda kv: -kv[1]["sum_us"]):
        out.append(f"  {c:<14s}{v['sum_us'] / 1e3:11.2f}{100 * v['sum_us'] / w:7.1f}%{v['launches']:10d}")
    if r["comm_overlap"] is not None:
        out.append(f"  communication overlapped with compute: {100 * r['comm_overlap']:.1f}% "
                   f"(exposed {r['comm_exposed_us'] / 1e3:.2f} ms)")
    if r.get("stages"):
        out.append("  stage (NVTX range at launch)   kernel ms  launches  communication ms  overlapped")
        for st, v in sorted(r["stages"].items()):
            ov = "-" if v["comm_overlap"] is None else f"{100 * v['comm_overlap']:.0f}%"
            out.append(f"  {st:<30s}{v['sum_us'] / 1e3:10.2f}{v['launches']:10d}{v['comm_us'] / 1e3:18.2f}{ov:>12s}")
    out.append("  top kernels         sum ms  launches   mean us  name")
    for k in r["top"]:
        out.append(f"  {k['sum_us'] / 1e3:17.2f}{k['launches']:10d}{k['mean_us']:10.1f}  {k['name'][:100]}")
    return out


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("path", type=Path, help="trace file (.json, .json.gz or an nsys .sqlite export) or a directory of them")
    ap.add_argument("--top", type=int, default=25)
    ap.add_argument("--json", type=Path, default=None)
    a = ap.parse_args(argv)
    files = [a.path] if a.path.is_file() else sorted(list(a.path.glob("trace_rank*.json.gz")) + list(a.path.glob("trace_rank*.json"))
                                                      + list(a.path.glob("*.sqlite")))
    if not files:
        print(f"no traces under {a.path}")
        return 1
    results = {}
    for f in files:
        events = load_events_sqlite(f) if f.suffix == ".sqlite" else load_events(f)
        results[f.name.split(".")[0]] = analyze_events(events, a.top)
    for rank, r in results.items():
        print("\n".join(render(rank, r)))
    if a.json:
        a.json.write_text(json.dumps(results, indent=1))
    return 0


if __name__ == "__main__":
    sys.exit(main())
