"""Build the native sm_100a library in-tree with nvcc (no torch headers, no JIT cache).

Every ``csrc/*.cu`` file is compiled to an object with
``-gencode arch=compute_100a,code=sm_100a -lineinfo`` and linked into
``pithtrain_b200/_lib/libpithb200.so``, which :mod:`pithtrain_b200._native` loads with ctypes.
Objects are rebuilt only when their source (or a header) is newer.
"""

from __future__ import annotations

import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

ROOT = Path(__file__).resolve().parent
CSRC = ROOT / "csrc"
LIBDIR = ROOT / "_lib"
LIBNAME = "libpithb200.so"

NVCC_FLAGS = [
    "-gencode",
    "arch=compute_100a,code=sm_100a",
    "-lineinfo",
    "-O3",
    "-std=c++17",
    "--use_fast_math",
    "-Xcompiler",
    "-fPIC",
    "-Xcompiler",
    "-fvisibility=hidden",
    "--expt-relaxed-constexpr",
]


def _nvcc() -> str:
    cand = os.environ.get("NVCC") or "/usr/local/cuda/bin/nvcc"
    return cand if os.path.exists(cand) else "nvcc"


def _newest_header_mtime() -> float:
    return max((p.stat().st_mtime for p in list(CSRC.glob("*.cuh")) + list(CSRC.glob("*.h"))), default=0.0)


def lib_path() -> Path:
    return LIBDIR / LIBNAME


def build(verbose: bool = False, force: bool = False, ptxas_info: bool = False, bounds_check: bool = False) -> Path:
    """Compile and link the library; returns its path. ``bounds_check`` builds ``libpithb200_checked.so`` with
    ``-DPT_BOUNDS_CHECK`` (index validation in the kernels that address memory through device-computed indices)."""
    LIBDIR.mkdir(exist_ok=True)
    objdir = LIBDIR / ("obj_checked" if bounds_check else "obj")
    objdir.mkdir(exist_ok=True)
    sources = sorted(CSRC.glob("*.cu"))
    hdr_m = _newest_header_mtime()
    jobs = []
    for src in sources:
        obj = objdir / (src.stem + ".o")
        stale = force or not obj.exists() or obj.stat().st_mtime < max(src.stat().st_mtime, hdr_m)
        if stale:
            cmd = [_nvcc(), *NVCC_FLAGS, *(["-DPT_BOUNDS_CHECK"] if bounds_check else []), "-c", str(src), "-o", str(obj)]
            if ptxas_info:
                cmd[1:1] = ["-Xptxas", "-v"]
            jobs.append((src, cmd))

    def run(job):
        src, cmd = job
        res = subprocess.run(cmd, capture_output=True, text=True)
        return src, res

    if jobs:
        with ThreadPoolExecutor(max_workers=min(8, len(jobs))) as ex:
            for src, res in ex.map(run, jobs):
                if verbose or ptxas_info or res.returncode != 0:
                    sys.stderr.write(f"[build] {src.name}\n{res.stdout}{res.stderr}\n")
                if res.returncode != 0:
                    raise RuntimeError(f"nvcc failed for {src}")
    out = LIBDIR / "libpithb200_checked.so" if bounds_check else lib_path()
    objs = [str(objdir / (s.stem + ".o")) for s in sources]
    need_link = bool(jobs) or not out.exists()
    if need_link:
        cmd = [_nvcc(), "-shared", "-o", str(out), *objs, "-lcudart_static", "-lrt", "-lpthread", "-ldl"]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            sys.stderr.write(res.stdout + res.stderr)
            raise RuntimeError("link failed")
    return out


if __name__ == "__main__":
    p = build(verbose=True, force="--force" in sys.argv, ptxas_info="--ptxas" in sys.argv,
              bounds_check="--bounds-check" in sys.argv)
    print(p)
