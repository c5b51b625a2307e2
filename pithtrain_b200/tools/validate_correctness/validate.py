"""Short deterministic training run whose rank-0 log is the input of ``compare.py``.

    torchrun --nproc-per-node 8 -m pithtrain_b200.tools.validate_correctness.validate \
        --model qwen3-30b-a3b --pipeline-parallel-size 2 --expert-parallel-size 4 > base.log

AdamW with a constant 1e-6 learning rate from the released step-0 checkpoint (or from the seeded random
init when no checkpoint exists), natural routing, bf16 — the recipe of the reference's check
(.agents/skills/validate-correctness/scripts/validate.py:1-60 of the reference). ``--synthetic`` replaces the
tokenized corpus with the seeded synthetic stream so the check also runs on a machine without data.
"""

from __future__ import annotations

import argparse
from pathlib import Path

from ...modules.training import make_adamw_optimizer, make_constant_scheduler
from ...tasks.pretrain_lm import PretrainLMCfg, launch

RECIPES = {
    "deepseek-v2-lite": ("deepseek-v2", "sequence", 3e-3),
    "qwen3-30b-a3b": ("qwen3", "global-batch", 1e-3),
    "gpt-oss-20b": ("gpt-oss", "global-batch", 1e-3),
    "qwen3.5-35b-a3b": ("qwen3.5", "global-batch", 1e-3),
}


def make_cfg(a: argparse.Namespace) -> PretrainLMCfg:
    tok, lb_type, lb_coef = RECIPES[a.model]
    cfg = PretrainLMCfg()
    cfg.distributed.pipeline_parallel_size = a.pipeline_parallel_size
    cfg.distributed.expert_parallel_size = a.expert_parallel_size
    cfg.distributed.context_parallel_size = a.context_parallel_size
    t = cfg.training
    t.model = Path(f"examples/pretrain_lm/{a.model}/config.json")
    t.dataset = None if a.synthetic else Path(f"workspace/datasets/dclm-baseline/toktxt/{tok}")
    t.optimizer, t.scheduler, t.lr = make_adamw_optimizer, make_constant_scheduler, 1e-6
    t.max_steps, t.micro_batch_size, t.global_batch_size = a.max_steps, 1, a.global_batch_size
    t.sequence_length = a.sequence_length
    t.moe_load_balance_type, t.moe_load_balance_coef = lb_type, lb_coef
    t.fp8 = a.fp8
    t.save_location = Path(f"workspace/checkpoints/{a.model}")
    t.save_interval = None
    if a.num_hidden_layers:
        t.num_hidden_layers_override = a.num_hidden_layers
    return cfg


def main(argv=None) -> None:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--model", required=True, choices=sorted(RECIPES))
    ap.add_argument("--pipeline-parallel-size", type=int, required=True)
    ap.add_argument("--expert-parallel-size", type=int, required=True)
    ap.add_argument("--context-parallel-size", type=int, default=1)
    ap.add_argument("--sequence-length", type=int, default=2048)
    ap.add_argument("--global-batch-size", type=int, default=1024)
    ap.add_argument("--max-steps", type=int, default=25)
    ap.add_argument("--num-hidden-layers", type=int, default=0, help="truncate the model (debugging only)")
    ap.add_argument("--synthetic", action="store_true")
    ap.add_argument("--fp8", action="store_true")
    launch(make_cfg(ap.parse_args(argv)))


if __name__ == "__main__":
    main()
