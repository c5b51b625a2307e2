"""One table row per Nsight Compute report: the counters a roofline argument needs, nothing else.

    python -m pithtrain_b200.tools.profile.ncu_table prof_gemm.ncu-rep prof_rmsnorm.ncu-rep ...      # runs `ncu -i ... --page raw --csv`
    python -m pithtrain_b200.tools.profile.ncu_table --csv raw_gemm.csv                               # an export made elsewhere

Per captured launch it prints the kernel name, duration, DRAM bytes read / written and DRAM throughput (% of peak), the
tensor-pipe and SM activity, registers per thread, dynamic shared memory, grid x block, L2 hit rate and the three
largest warp-stall reasons, as a Markdown table (the format of the summaries under ``profiles/``). Given the
algorithmic bytes or FLOPs of the launch (``--bytes`` / ``--flops``) it adds the achieved fraction of the measured
peaks (``MEASURED_PEAKS.json`` at the repository root when present). Reports are read, never captured, by this tool:
captures are made with ``ncu --set full --clock-control none -k regex:<kernel> -c 1..3`` on a small case.
"""

from __future__ import annotations

import argparse
import csv
import io
import json
import subprocess
import sys
from pathlib import Path
from typing import Dict, List, Optional, Tuple

WANT = {
    "gpu__time_duration.sum": "time",
    "dram__bytes_read.sum": "dram_rd",
    "dram__bytes_write.sum": "dram_wr",
    "gpu__dram_throughput.avg.pct_of_peak_sustained_elapsed": "dram_pct",
    "sm__pipe_tensor_cycles_active.avg.pct_of_peak_sustained_active": "tensor_pct",
    "sm__throughput.avg.pct_of_peak_sustained_elapsed": "sm_pct",
    "launch__registers_per_thread": "regs",
    "launch__shared_mem_per_block_dynamic": "smem_dyn",
    "launch__grid_size": "grid",
    "launch__block_size": "block",
    "lts__t_sector_hit_rate.pct": "l2_hit",
}
STALL_PREFIX, STALL_SUFFIX = "smsp__average_warps_issue_stalled_", "_per_issue_active.ratio"
TIME_UNITS = {"ns": 1e-9, "us": 1e-6, "usecond": 1e-6, "ms": 1e-3, "msecond": 1e-3, "s": 1.0, "second": 1.0, "nsecond": 1e-9}


def parse_raw_csv(text: str) -> List[Dict[str, Tuple[str, str]]]:
    """Rows of ``ncu --page raw --csv``: a header line, a units line, then one line per captured launch."""
    rows = [r for r in csv.reader(io.StringIO(text)) if r]
    start = next((i for i, r in enumerate(rows) if "Kernel Name" in r), None)
    if start is None or len(rows) < start + 3:
        return []
    header, units = rows[start], rows[start + 1]
    out = []
    for vals in rows[start + 2:]:
        d: Dict[str, Tuple[str, str]] = {}
        stalls = []
        for h, u, v in zip(header, units, vals):
            if h in WANT:
                d[WANT[h]] = (v, u)
            elif h == "Kernel Name":
                d["kernel"] = (v, "")
            elif h.startswith(STALL_PREFIX) and h.endswith(STALL_SUFFIX):
                try:
                    stalls.append((float(v.replace(",", "")), h[len(STALL_PREFIX):-len(STALL_SUFFIX)]))
                except ValueError:
                    pass
        stalls.sort(reverse=True)
        d["stalls"] = (", ".join(f"{n} {x:.1f}" for x, n in [s for s in stalls if s[1] != "selected"][:3]), "")
        out.append(d)
    return out


def _number(cell: Optional[Tuple[str, str]], units: Dict[str, float]) -> Optional[float]:
    if cell is None:
        return None
    try:
        return float(cell[0].replace(",", "")) * units.get(cell[1], 1.0)
    except ValueError:
        return None


def load_report(path: Path) -> List[Dict[str, Tuple[str, str]]]:
    if path.suffix == ".csv":
        return parse_raw_csv(path.read_text())
    res = subprocess.run(["ncu", "-i", str(path), "--page", "raw", "--csv"], capture_output=True, text=True)
    if res.returncode != 0:
        raise SystemExit(f"ncu could not read {path}: {res.stderr.strip()[:200]}")
    return parse_raw_csv(res.stdout)


def peaks(root: Path) -> Dict[str, float]:
    p = root / "MEASURED_PEAKS.json"
    if p.exists():
        return json.loads(p.read_text())
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "fallback": True}


HEADER = ("| report | kernel | time | DRAM read / written | DRAM % | tensor % | SM % | regs / dyn smem | grid x block | L2 hit % | "
          "top stalls | of peak |")


def table(reports: List[Tuple[str, Dict[str, Tuple[str, str]]]], alg_bytes: Optional[float], flops: Optional[float],
          pk: Dict[str, float]) -> List[str]:
    lines = [HEADER, "|" + "---|" * 12]
    for name, d in reports:
        g = lambda k: " ".join(x for x in d.get(k, ("?", "")) if x)  # noqa: E731
        seconds = _number(d.get("time"), TIME_UNITS)
        frac = "-"
        tag = "of fallback" if pk.get("fallback") else "of measured"
        if seconds and alg_bytes:
            frac = f"{alg_bytes / seconds / 1e9 / pk['hbm_gbs']:.2f} {tag} HBM"
        elif seconds and flops:
            frac = f"{flops / seconds / 1e12 / pk['bf16_tflops']:.2f} {tag} bf16"
        lines.append(f"| {name} | {d.get('kernel', ('?', ''))[0][:60]} | {g('time')} | {g('dram_rd')} / {g('dram_wr')} | {g('dram_pct')} | "
                     f"{g('tensor_pct')} | {g('sm_pct')} | {g('regs')} / {g('smem_dyn')} | {g('grid')} x {g('block')} | {g('l2_hit')} | "
                     f"{d.get('stalls', ('', ''))[0]} | {frac} |")
    return lines


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("reports", nargs="*", type=Path, help=".ncu-rep files (read through `ncu -i`) or raw-page .csv exports")
    ap.add_argument("--csv", type=Path, action="append", default=[], help="a raw-page CSV export")
    ap.add_argument("--bytes", type=float, default=None, help="algorithmic bytes of one launch: adds the fraction of the HBM peak")
    ap.add_argument("--flops", type=float, default=None, help="FLOPs of one launch: adds the fraction of the bf16 GEMM peak")
    a = ap.parse_args(argv)
    rows: List[Tuple[str, Dict[str, Tuple[str, str]]]] = []
    for path in list(a.reports) + list(a.csv):
        for i, d in enumerate(load_report(path)):
            rows.append((path.stem if i == 0 else f"{path.stem} #{i + 1}", d))
    if not rows:
        print("no captured launches found")
        return 1
    root = Path(__file__).resolve().parents[3]
    print("\n".join(table(rows, a.bytes, a.flops, peaks(root))))
    return 0


if __name__ == "__main__":
    sys.exit(main())
