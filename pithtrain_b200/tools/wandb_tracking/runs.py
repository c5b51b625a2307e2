"""List the runs of a project, compare a logged metric between runs step by step, download run files.

    python -m pithtrain_b200.tools.wandb_tracking.runs list    <entity/project>
    python -m pithtrain_b200.tools.wandb_tracking.runs compare <entity/project> --metric train/cross-entropy-loss \\
        --ref <run> --runs <run>[,<run>...] [--skip-steps N]
    python -m pithtrain_b200.tools.wandb_tracking.runs files   <entity/project> --runs <run>[,...] [--file output.log] [--out DIR]

``<run>`` is a run id or its display name. ``compare`` prints, per run, the range and the mean of the per-step
difference to the reference run over the common steps, and the difference at the last common step — facts, not a
verdict. Metrics are the ones the trainer logs (``train/cross-entropy-loss``, ``train/load-balance-loss``,
``train/gradient-norm``, ``infra/tokens-per-second``, ``infra/peak-gpu-memory``, ``infra/step-time``).
The wandb client is imported lazily; ``main(argv, api=...)`` takes any object with the client's ``runs(path)`` /
``run(path)`` interface, which is how the tests drive it. Same job as the reference's helper
(.agents/skills/wandb-tracking/scripts/runs.py).
"""

from __future__ import annotations

import argparse
import statistics
import sys
from pathlib import Path
from typing import Dict, List, Optional


def _api():
    try:
        import wandb
    except ImportError as e:  # pragma: no cover - depends on the environment
        raise SystemExit("the wandb client is not installed in this environment (pip install wandb)") from e
    return wandb.Api()


def resolve(api, project: str, selector: str):
    """Run object for an id or a display name."""
    runs = list(api.runs(project))
    by_id = {r.id: r for r in runs}
    if selector in by_id:
        return by_id[selector]
    named = [r for r in runs if r.name == selector]
    if len(named) == 1:
        return named[0]
    if not named:
        raise SystemExit(f"no run {selector!r} in {project}")
    raise SystemExit(f"{len(named)} runs are called {selector!r} in {project}: use the id ({', '.join(r.id for r in named)})")


def metric_series(run, key: str) -> Dict[int, float]:
    out: Dict[int, float] = {}
    for row in run.scan_history(keys=["_step", key]):
        v = row.get(key)
        if v is not None:
            out[int(row["_step"])] = float(v)
    return out


def cmd_list(api, project: str) -> List[str]:
    runs = sorted(api.runs(project), key=lambda r: r.name)
    lines = [f"{project}: {len(runs)} runs", f"{'id':<12}{'state':<10}{'steps':>8}  name"]
    for r in runs:
        steps = getattr(r, "lastHistoryStep", None)
        lines.append(f"{r.id:<12}{r.state:<10}{(steps if steps is not None else '-'):>8}  {r.name}")
    return lines


def cmd_compare(api, project: str, metric: str, ref: str, others: List[str], skip_steps: int = 0) -> List[str]:
    base_run = resolve(api, project, ref)
    base = metric_series(base_run, metric)
    lines = [f"{metric}: reference {base_run.name} ({len(base)} steps)"]
    for sel in others:
        run = resolve(api, project, sel)
        cur = metric_series(run, metric)
        steps = sorted(s for s in set(base) & set(cur) if s >= skip_steps)
        if not steps:
            lines.append(f"  {run.name}: no common steps")
            continue
        diff = [cur[s] - base[s] for s in steps]
        rel = [abs(d) / max(abs(base[s]), 1e-12) for d, s in zip(diff, steps)]
        lines.append(f"  {run.name}: {len(steps)} common steps; difference min {min(diff):+.5g} max {max(diff):+.5g} "
                     f"mean {statistics.fmean(diff):+.5g}; largest relative {max(rel):.3e}; at step {steps[-1]}: {diff[-1]:+.5g}")
    return lines


def cmd_files(api, project: str, selectors: List[str], name: str, out: Path) -> List[str]:
    lines = []
    for sel in selectors:
        run = resolve(api, project, sel)
        dest = out / run.name
        dest.mkdir(parents=True, exist_ok=True)
        run.file(name).download(root=str(dest), replace=True)
        lines.append(f"{run.name}: {name} -> {dest / name}")
    return lines


def main(argv: Optional[List[str]] = None, api=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    sub = ap.add_subparsers(dest="cmd", required=True)
    p = sub.add_parser("list"); p.add_argument("project")
    p = sub.add_parser("compare"); p.add_argument("project")
    p.add_argument("--metric", required=True); p.add_argument("--ref", required=True); p.add_argument("--runs", required=True)
    p.add_argument("--skip-steps", type=int, default=0, help="leave the first N steps out (warm-up outliers of throughput metrics)")
    p = sub.add_parser("files"); p.add_argument("project")
    p.add_argument("--runs", required=True); p.add_argument("--file", default="output.log")
    p.add_argument("--out", type=Path, default=Path("workspace/wandb-logs"))
    a = ap.parse_args(argv)
    api = api or _api()
    if a.cmd == "list":
        lines = cmd_list(api, a.project)
    elif a.cmd == "compare":
        lines = cmd_compare(api, a.project, a.metric, a.ref, [s for s in a.runs.split(",") if s], a.skip_steps)
    else:
        lines = cmd_files(api, a.project, [s for s in a.runs.split(",") if s], a.file, a.out)
    print("\n".join(lines))
    return 0


if __name__ == "__main__":
    sys.exit(main())
