"""Command line of the memory estimator.

    python -m pithtrain_b200.tools.memory_estimator --model examples/pretrain_lm/qwen3-30b-a3b/config.json \
        --pp-size 2 --ep-size 4 --total-gpus 8 --micro-batch-size 1 --global-batch-size 256 --sequence-length 4096

Flags mirror the reference's estimator (tools/memory_estimator/__main__.py:1-19 of the reference): ``--detail``,
``--timeline``, ``--timeline-limit``, ``--pp-rank``, ``--ep-imbalance``, ``--fragmentation``, ``--gpu-memory-gb``.
"""

from __future__ import annotations

import argparse
import sys

from .model_profile import ModelDims, ParallelCfg
from .report import detail_lines, suggestion_lines, summary_lines, timeline_lines, verdict
from .schedule_simulator import estimate


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="pithtrain_b200.tools.memory_estimator", description=__doc__.split("\n")[0])
    ap.add_argument("--model", required=True, help="Hugging Face style config.json")
    ap.add_argument("--pp-size", type=int, default=1)
    ap.add_argument("--ep-size", type=int, default=1)
    ap.add_argument("--cp-size", type=int, default=1)
    ap.add_argument("--total-gpus", type=int, default=0, help="0 = pp·ep·cp (dp = 1)")
    ap.add_argument("--micro-batch-size", type=int, default=1)
    ap.add_argument("--global-batch-size", type=int, default=32)
    ap.add_argument("--sequence-length", type=int, default=4096)
    ap.add_argument("--gpu-memory-gb", type=float, default=192.0, help="B200: 183,359 MiB = 192 GB")
    ap.add_argument("--grad-dtype", choices=["bf16", "fp32"], default="bf16")
    ap.add_argument("--optimizer", choices=["muon", "adamw"], default="muon")
    ap.add_argument("--momentum-dtype", choices=["bf16", "fp32"], default="bf16")
    ap.add_argument("--offload-optimizer-state", action="store_true")
    ap.add_argument("--reshard-params", action="store_true", help="DistributedCfg.reshard_params (parameters sharded between steps)")
    ap.add_argument("--resident-state-gb", type=float, default=0.0, help="with offload: GiB of optimizer state kept on the device")
    ap.add_argument("--ep-backend", choices=["fused", "nccl"], default="fused")
    ap.add_argument("--fp8-training", action="store_true", help="TrainingCfg.fp8: adds the cached e4m3 weight copies")
    ap.add_argument("--pp-rank", type=int, default=-1, help="-1 = report the worst rank")
    ap.add_argument("--ep-imbalance", type=float, default=1.0)
    ap.add_argument("--fragmentation", type=float, default=0.05)
    ap.add_argument("--detail", action="store_true")
    ap.add_argument("--timeline", action="store_true")
    ap.add_argument("--timeline-limit", type=int, default=100)
    a = ap.parse_args(argv)

    inner = a.pp_size * a.ep_size * a.cp_size
    total = a.total_gpus or inner
    if total % inner:
        ap.error(f"--total-gpus {total} is not a multiple of pp·ep·cp = {inner}")
    par = ParallelCfg(pp=a.pp_size, ep=a.ep_size, cp=a.cp_size, dp=total // inner, micro_batch_size=a.micro_batch_size,
                      global_batch_size=a.global_batch_size, sequence_length=a.sequence_length, grad_dtype=a.grad_dtype,
                      optimizer=a.optimizer, momentum_dtype=a.momentum_dtype,
                      offload_optimizer_state=a.offload_optimizer_state, resident_state_gb=a.resident_state_gb,
                      reshard_params=a.reshard_params,
                      ep_backend=a.ep_backend, fp8_training=a.fp8_training)
    dims = ModelDims.from_json(a.model)
    ranks = [a.pp_rank] if a.pp_rank >= 0 else list(range(par.pp))
    ests = {r: estimate(dims, par, r, a.ep_imbalance, a.fragmentation, keep_timeline=a.timeline) for r in ranks}
    worst = max(ests, key=lambda r: ests[r].peak_total)
    est = ests[worst]
    print("\n".join(summary_lines(est, dims, par, worst, a.gpu_memory_gb)))
    if len(ests) > 1:
        print("  per pp rank: " + ", ".join(f"{r}: {ests[r].peak_total / 1024 ** 3:.1f} GiB" for r in ranks))
    if a.detail:
        print("\n" + "\n".join(detail_lines(dims, par, worst, est)))
    if a.timeline:
        print("\n" + "\n".join(timeline_lines(est, a.timeline_limit)))
    s = suggestion_lines(est, par, a.gpu_memory_gb)
    if s:
        print("\n" + "\n".join(s))
    return 0 if verdict(est.peak_total, a.gpu_memory_gb) != "OOM" else 1


if __name__ == "__main__":
    sys.exit(main())
