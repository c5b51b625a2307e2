"""Compare two training logs: losses must agree step by step, speed and memory are reported.

    python -m pithtrain_b200.tools.validate_correctness.compare base.log feature.log [--tolerance 5e-3]

A step line is what the trainer's rank-0 logger prints: ``step 00000003/00000025 | step-time 6.9 sec |
cross-entropy-loss 12.33 | ...``; every ``name value [unit]`` field is picked up. Exit status 1 when a loss
differs by more than the relative tolerance at any step (default 5e-3, the gate of
.agents/skills/validate-correctness/scripts/compare.py:8-9 of the reference), or when the logs cover different steps.
"""

from __future__ import annotations

import argparse
import re
import statistics
import sys
from typing import Dict, List, Tuple

GATED = ("cross-entropy-loss", "load-balance-loss")
REPORTED = ("step-time", "device-step-time", "tokens-per-second", "peak-gpu-memory")
_STEP = re.compile(r"\bstep (\d+)/(\d+)")
_FIELD = re.compile(r"^([A-Za-z][A-Za-z0-9\-_ ]*?)\s+(-?[0-9][0-9,]*\.?[0-9]*(?:[eE][-+]?\d+)?|nan|inf)\b")


def parse_log(path: str) -> Dict[int, Dict[str, float]]:
    rows: Dict[int, Dict[str, float]] = {}
    with open(path, errors="replace") as f:
        for line in f:
            m = _STEP.search(line)
            if not m:
                continue
            fields: Dict[str, float] = {}
            for part in line[m.end():].split("|"):
                fm = _FIELD.match(part.strip())
                if fm:
                    fields[fm.group(1).strip()] = float(fm.group(2).replace(",", ""))
            if fields:
                rows[int(m.group(1))] = fields
    return rows


def loss_mismatches(a: Dict[int, Dict[str, float]], b: Dict[int, Dict[str, float]], tol: float) -> List[str]:
    bad: List[str] = []
    if set(a) != set(b):
        only_a, only_b = sorted(set(a) - set(b)), sorted(set(b) - set(a))
        bad.append(f"step sets differ: only in base {only_a[:5]}, only in feature {only_b[:5]}")
    for step in sorted(set(a) & set(b)):
        for name in GATED:
            x, y = a[step].get(name), b[step].get(name)
            if x is None and y is None:
                continue
            if x is None or y is None:
                bad.append(f"step {step}: {name} is logged by one run only")
                continue
            if x != x or y != y:  # NaN never passes
                bad.append(f"step {step}: {name} is NaN (base {x}, feature {y})")
                continue
            scale = max(abs(x), abs(y))
            if scale and abs(x - y) / scale > tol:
                bad.append(f"step {step}: {name} base {x:.6f} vs feature {y:.6f} (rel {abs(x - y) / scale:.2e} > {tol:.0e})")
    return bad


def steady(values: List[float], skip: int) -> Tuple[float, float]:
    v = values[skip:] or values
    return statistics.median(v), (statistics.pstdev(v) if len(v) > 1 else 0.0)


def report(a, b, skip: int) -> List[str]:
    out = [f"{'metric':<22s}{'base':>14s}{'feature':>14s}{'change':>10s}"]
    steps = sorted(set(a) & set(b))
    for name in REPORTED:
        va = [a[s][name] for s in steps if name in a[s]]
        vb = [b[s][name] for s in steps if name in b[s]]
        if not va or not vb:
            continue
        (ma, _), (mb, _) = steady(va, skip), steady(vb, skip)
        out.append(f"{name:<22s}{ma:14.3f}{mb:14.3f}{(mb / ma - 1) * 100 if ma else 0:+9.1f}%")
    return out


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("base")
    ap.add_argument("feature")
    ap.add_argument("--tolerance", type=float, default=5e-3)
    ap.add_argument("--skip", type=int, default=3, help="warm-up steps left out of the speed medians")
    a = ap.parse_args(argv)
    base, feat = parse_log(a.base), parse_log(a.feature)
    if not base or not feat:
        print("no step lines found in " + (a.base if not base else a.feature))
        return 1
    bad = loss_mismatches(base, feat, a.tolerance)
    print(f"{len(set(base) & set(feat))} common steps; losses gated at rel {a.tolerance:.0e}")
    print("\n".join(report(base, feat, a.skip)))
    if bad:
        print("MISMATCH\n  " + "\n  ".join(bad[:40]))
        return 1
    print("losses agree")
    return 0


if __name__ == "__main__":
    sys.exit(main())
