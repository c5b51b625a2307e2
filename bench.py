"""Headline benchmark: Qwen3-30B-A3B-architecture pre-training at sequence length 4096.

    python bench.py --gpus N --steps K --warmup W          (N > 1: launched through torchrun)

Runs the flagship training step through the public task API (``PretrainLMCfg`` -> ``setup_*`` ->
``forward_backward_update`` / ``train_step``) on synthetic uniform token ids with random-init
weights, weak-scaled at 32 sequences of 4096 tokens per GPU per optimizer step (the 8-GPU job is
the 1M-token global batch). Two timed regions of K steps each, both bracketed by a barrier and a
device synchronize and timed with CUDA events (max over ranks):

* ``value``: inputs already on the device, nothing read back (forward + backward of every
  micro-batch, gradient reduction, clipping, Muon/AdamW step, parameter all-gather);
* ``e2e``: ``train_step`` as a user calls it — token ids copied from pinned host memory every step
  and the loss read back to the host.

Prints one JSON line on rank 0. ``--impl reference`` reports on the reference arm.
"""

from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

SEQ_LEN = 4096
SEQS_PER_GPU = 32
MODEL = "Qwen/Qwen3-30B-A3B"
METRIC = "tokens/sec (whole job), Qwen3-30B-A3B arch seq 4096"


def parallelism_for(n: int, override: str | None):
    """(pp, cp, ep) for N GPUs. 8 GPUs use the PP2 x EP4 layout named by the benchmark config."""
    if override:
        parts = dict(pp=1, cp=1, ep=1)
        for tok in override.replace("x", ",").split(","):
            tok = tok.strip()
            for k in parts:
                if tok.startswith(k):
                    parts[k] = int(tok[len(k):])
        return parts["pp"], parts["cp"], parts["ep"]
    return {1: (1, 1, 1), 2: (1, 1, 2), 4: (1, 1, 4), 8: (2, 1, 4)}.get(n, (1, 1, n))


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.rows, self.proc = index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "200",
                 "-i", str(self.index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([x.strip() for x in line.split(",")])

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        sm, mx, reasons = [], [], set()
        for r in self.rows:
            try:
                sm.append(float(r[0])); mx.append(float(r[1]))
            except Exception:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), r[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        sm.sort()
        # median over samples under load (clocks above idle)
        load = [x for x in sm if x > 0.5 * (mx[0] if mx else 1)] or sm
        med = load[len(load) // 2] if load else None
        return {"sm_mhz": med, "sm_max_mhz": (mx[0] if mx else None), "reasons": sorted(reasons), "samples": len(sm)}


def reference_arm(args) -> int:
    """The reference cannot run here: say why in one line."""
    why = ("reference build unavailable on this box: pithtrain 0.1.3 needs deep-gemm (git), flash-attn-4[cu13], "
           "torch>=2.12 / CUDA 13; none is in the offline wheelhouse (pip install --no-index fails at dependency "
           "resolution, --no-deps installs a package that raises ModuleNotFoundError: deep_gemm on import)")
    probe = ROOT / "baseline" / "_ref" / "pithtrain"
    if probe.exists():
        sys.path.insert(0, str(ROOT / "baseline" / "_ref"))
        try:
            import pithtrain.tasks.pretrain_lm  # noqa: F401
            why = "reference imported but its CUDA>=13 / FA4 / DeepGEMM code path is not runnable with torch 2.11+cu128"
        except Exception as e:  # the expected outcome
            why = f"reference installed with --no-deps but not importable: {type(e).__name__}: {str(e)[:160]}"
    if int(os.environ.get("RANK", "0")) == 0:
        print(json.dumps({"impl": "reference", "unavailable": why}))
    return 0


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours")
    ap.add_argument("--parallelism", default=os.environ.get("PITH_BENCH_PARALLELISM"))
    ap.add_argument("--layers", type=int, default=None, help="debug only: truncate the model (result is marked invalid)")
    ap.add_argument("--seqs-per-gpu", type=int, default=SEQS_PER_GPU)
    ap.add_argument("--optimizer", default="muon")
    ap.add_argument("--resident-state-gb", type=float, default=22.0,
                    help="N=1 only: GiB of Muon momentum kept on the device, the rest streams from pinned host memory")
    ap.add_argument("--state-dtype", choices=["auto", "fp32", "bf16"], default="auto",
                    help="gradient accumulators and Muon momentum: auto = fp32 from 2 GPUs on (the reference's precision), bf16 on one GPU")
    ap.add_argument("--pair-wgrads", action="store_true",
                    help="expert weight gradients of two micro-batches per launch (TrainingCfg.pair_expert_wgrads); off: with worst-case "
                         "sized expert-parallel buffers the operands held for the partner micro-batch do not fit at this batch size")
    ap.add_argument("--fp8", action="store_true", help="not the headline run: forward/dgrad GEMMs in block-scaled e4m3 (dtype says so)")
    ap.add_argument("--ep-backend", default=os.environ.get("PITH_EP_BACKEND", "auto"))
    ap.add_argument("--routing", choices=["natural", "balanced"], default="natural",
                    help="balanced = TrainingCfg.benchmark: the round-robin router replay of the reference's throughput recipes")
    args = ap.parse_args()
    if args.impl == "reference":
        return reference_arm(args)
    args.warmup = max(args.warmup, 3)

    os.environ.setdefault("PYTORCH_CUDA_ALLOC_CONF", "expandable_segments:True")
    import torch
    import torch.distributed as dist

    from pithtrain_b200 import _native
    from pithtrain_b200.contexts import distributed, training
    from pithtrain_b200.modules.distributed import setup_distributed
    from pithtrain_b200.modules.logging import setup_logging
    from pithtrain_b200.modules.training import (make_adamw_optimizer, make_constant_scheduler, make_muon_optimizer,
                                                 setup_training)
    from pithtrain_b200.tasks.pretrain_lm import (PretrainLMCfg, forward_backward_update, get_global_batch,
                                                  model_flops_per_token, train_step)

    world = int(os.environ.get("WORLD_SIZE", "1"))
    n = world
    pp, cp, ep = parallelism_for(n, args.parallelism)
    cfg = PretrainLMCfg()
    cfg.distributed.pipeline_parallel_size, cfg.distributed.context_parallel_size = pp, cp
    cfg.distributed.expert_parallel_size = ep
    cfg.distributed.ep_backend = args.ep_backend
    t = cfg.training
    t.model = MODEL
    t.sequence_length = SEQ_LEN
    t.micro_batch_size = 1
    t.global_batch_size = args.seqs_per_gpu * n
    t.lr, t.max_steps = 1.0e-6, 1 << 30
    t.optimizer = make_muon_optimizer if args.optimizer == "muon" else make_adamw_optimizer
    t.scheduler = make_constant_scheduler
    t.dataset = None  # synthetic uniform token ids
    # Optimizer-state precision: the reference accumulates gradients and keeps Muon momentum in fp32
    # (pithtrain/modules/training.py:349-354, modules/optimizer.py:193-200). The benchmark does the same wherever the
    # state fits in 180 GB per GPU and says what it ran in "config":
    #   N >= 4: fp32 gradient accumulators and fp32 momentum;
    #   N = 2 : fp32 accumulators (64 GB per GPU) and bf16 momentum (fp32 momentum, 58 GB more, does not fit);
    #   N = 1 : bf16 accumulators and bf16 momentum (61 GB of parameters + 122 GB of fp32 gradients exceed one GPU).
    if args.state_dtype == "auto":
        grads_wide, mom_wide = n >= 2, n >= 4
    else:
        grads_wide = mom_wide = args.state_dtype == "fp32"
    t.grad_dtype = "fp32" if grads_wide else "bf16"
    t.fp8 = bool(args.fp8)
    t.muon_momentum_dtype = "fp32" if mom_wide else "bf16"
    t.offload_optimizer_state = (n == 1)  # the 30B model + gradients fill one 180 GB GPU
    t.optimizer_device_state_gb = args.resident_state_gb if n == 1 else 0.0  # spare HBM keeps part of it resident
    t.pair_expert_wgrads = bool(args.pair_wgrads)
    t.num_hidden_layers_override = args.layers
    t.benchmark = args.routing == "balanced"

    setup_logging(cfg)
    setup_distributed(cfg, failfast=True)  # a rank that dies (e.g. out of memory) takes the job down at once
    setup_training(cfg)
    dev = distributed.device
    rank = distributed.rank

    def barrier_sync():
        if dist.is_initialized() and world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(x: float) -> float:
        v = torch.tensor([x], device=dev, dtype=torch.float64)
        if dist.is_initialized() and world > 1:
            dist.all_reduce(v, op=dist.ReduceOp.MAX)
        return float(v.item())

    # ---- warm-up (also builds pinned buffers, optimizer state, symmetric buffers)
    for _ in range(args.warmup):
        train_step(cfg)

    sampler = ClockSampler(distributed.local_rank)
    if rank == 0:
        sampler.start()

    # ---- region 1: device-only
    staged = [get_global_batch(cfg, dev) for _ in range(1)]
    barrier_sync()
    _native.LAUNCHES = 0
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(args.steps):
        tok, lab = staged[0]
        forward_backward_update(cfg, tok, lab)
        training.step += 1
    e1.record()
    barrier_sync()
    launches = _native.LAUNCHES
    dev_ms = max_over_ranks(e0.elapsed_time(e1)) / args.steps

    # ---- region 2: end to end through train_step (host batch -> device, loss -> host)
    barrier_sync()
    e2, e3 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    w0 = time.time()
    e2.record()
    last = None
    for i in range(args.steps):
        last = train_step(cfg)
    e3.record()
    barrier_sync()
    wall_ms = max_over_ranks((time.time() - w0) * 1e3) / args.steps
    e2e_ms = max(max_over_ranks(e2.elapsed_time(e3)) / args.steps, wall_ms)
    clocks = sampler.stop() if rank == 0 else None

    _native.check_status()
    tokens_per_step = t.global_batch_size * SEQ_LEN
    value = tokens_per_step / (dev_ms / 1e3)
    e2e_value = tokens_per_step / (e2e_ms / 1e3)
    local_rows = t.global_batch_size // (distributed.dp_size * distributed.ep_size)
    h2d = 2 * local_rows * (SEQ_LEN // cp) * 8 if distributed.pp_rank == 0 else 0
    try:
        flops_tok = model_flops_per_token(training.model_config, SEQ_LEN)
    except Exception:
        flops_tok = None
    peaks = {}
    try:
        peaks = json.load(open(ROOT / "MEASURED_PEAKS.json"))
    except Exception:
        pass
    peak_tf = peaks.get("bf16_tflops_sustained", 1385.3)
    mfu = (value / n) * flops_tok / (peak_tf * 1e12) if flops_tok else None
    if rank == 0:
        out = {
            "metric": METRIC, "value": value, "unit": "tokens/s", "n_gpus": n, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": dev_ms, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": ("fp8 e4m3 block-scaled forward/dgrad GEMMs, bf16 elsewhere" if args.fp8 else "bf16"), "data": "synthetic uniform token ids, random-init N(0,0.02) weights",
            "tokens_per_sec_per_gpu": value / n, "mfu_of_measured_sustained_bf16": mfu,
            "config": {
                "model": "Qwen3-30B-A3B architecture (48 layers, hidden 2048, 32q/4kv heads x128, 128 experts top-8, "
                         "moe_intermediate 768, vocab 151936)" + ("" if args.layers is None else f" TRUNCATED to {args.layers} layers: INVALID"),
                "global_batch": t.global_batch_size, "global_batch_tokens": tokens_per_step, "seq_len": SEQ_LEN,
                "micro_batch": 1, "parallelism": f"pp{pp}xcp{cp}xep{ep}xdp{distributed.dp_size}",
                "optimizer": "Muon (2-D/expert weights) + AdamW (rest), grad clip 1.0" if args.optimizer == "muon" else "AdamW",
                "grad_accumulators": t.grad_dtype, "paired_expert_wgrads": t.pair_expert_wgrads, "muon_momentum": t.muon_momentum_dtype + (f", {t.optimizer_device_state_gb:.0f} GiB resident + the rest in pinned host memory (streamed each step)" if t.offload_optimizer_state else ""),
                "routing": ("natural (seeded random-init gate)" if args.routing == "natural"
                            else "force-balanced round-robin replay (benchmark mode)"), "ep_transport": args.ep_backend,
                "l2": "inputs larger than L2: every step streams >10 GB of parameters and activations, no explicit flush",
                "switches": {k: v for k, v in sorted(os.environ.items()) if k.startswith("PITHTRAIN_")},
            },
            "clocks": clocks,
            "e2e": {"value": e2e_value, "unit": "tokens/s", "ms_per_step": e2e_ms, "h2d_bytes_per_step": h2d,
                    "d2h_bytes_per_step": 8, "loss": (last or {}).get("loss")},
            "gpu_launches": launches,
        }
        print(json.dumps(out))
    if dist.is_initialized():
        dist.barrier()
    return 0


if __name__ == "__main__":
    sys.exit(main())
