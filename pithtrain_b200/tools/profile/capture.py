"""Record one steady-state training step of any pre-training script.

    torchrun --nproc-per-node 8 -m pithtrain_b200.tools.profile.capture examples/pretrain_lm/qwen3-30b-a3b/script.py \
        --warmup 5 --out workspace/profiles/qwen3

The script must expose ``make_cfg()`` or a module-level ``cfg`` (every script under ``examples/`` does). The
job is set up exactly as ``launch`` does, runs ``--warmup`` untimed steps, then one step under the profiler;
each rank writes ``<out>/trace_rank<r>.json.gz`` (Chrome trace format) and rank 0 prints where. The
reference drives ``nsys`` with 5 warm-up steps and one captured step for the same purpose
(.agents/skills/capture-nsys-profile/scripts/capture.py:66-67 of the reference); this tool needs nothing but
PyTorch. Numbers read from a trace are for attribution only: the profiler slows the step down.
"""

from __future__ import annotations

import argparse
import importlib.util
from pathlib import Path


def load_cfg(script: str):
    spec = importlib.util.spec_from_file_location("_profiled_script", script)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)  # scripts guard launch() behind __main__
    if hasattr(mod, "make_cfg"):
        return mod.make_cfg()
    if hasattr(mod, "cfg"):
        return mod.cfg
    raise SystemExit(f"{script} defines neither make_cfg() nor cfg")


def main(argv=None) -> None:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("script")
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--out", type=Path, default=Path("workspace/profiles/step"))
    ap.add_argument("--with-cpu", action="store_true",
                    help="also record CPU-side operator and launch events and the engine's stage ranges (per-stage table)")
    ap.add_argument("--synthetic", action="store_true", help="ignore the script's dataset and use the synthetic stream")
    a = ap.parse_args(argv)

    import torch
    from torch.profiler import ProfilerActivity, profile

    from ...contexts import distributed
    from ...modules.distributed import setup_distributed
    from ...modules.logging import setup_logging
    from ...modules.training import setup_training
    from ...tasks.pretrain_lm import load_checkpoint, train_step

    cfg = load_cfg(a.script)
    cfg.training.max_steps = 1 << 30
    cfg.training.save_interval = None
    if a.synthetic:
        cfg.training.dataset = None
    setup_logging(cfg)
    setup_distributed(cfg)
    setup_training(cfg)
    load_checkpoint(cfg)
    for _ in range(a.warmup):
        train_step(cfg)
    torch.cuda.synchronize()
    if a.with_cpu:
        from ...dualpipe import execution

        execution.RECORD_RANGES = True  # stage ranges become annotations the analysis can attribute kernels to
    acts = [ProfilerActivity.CUDA] + ([ProfilerActivity.CPU] if a.with_cpu else [])
    with profile(activities=acts) as prof:
        with torch.profiler.record_function("profiled_step"):
            train_step(cfg)
        torch.cuda.synchronize()
    a.out.mkdir(parents=True, exist_ok=True)
    path = a.out / f"trace_rank{distributed.rank}.json.gz"
    prof.export_chrome_trace(str(path))
    if distributed.rank == 0:
        print(f"wrote {distributed.world_size} trace(s) under {a.out}; analyse with "
              f"`python -m pithtrain_b200.tools.profile.analyze {a.out}`", flush=True)


if __name__ == "__main__":
    main()
