"""Pre-train Qwen3.5-35B-A3B: pipeline x1, expert x8, context x1; the data-parallel width is whatever is left."""

from functools import partial
from pathlib import Path

from pithtrain_b200.modules.training import make_muon_optimizer, make_wsd_scheduler
from pithtrain_b200.tasks.pretrain_lm import PretrainLMCfg, launch

HERE = Path(__file__).resolve().parent


def make_cfg() -> PretrainLMCfg:
    cfg = PretrainLMCfg()

    mesh = cfg.distributed
    mesh.pipeline_parallel_size = 1
    mesh.expert_parallel_size = 8
    mesh.context_parallel_size = 1

    t = cfg.training
    t.model = HERE / "config.json"
    t.dataset = Path("workspace/datasets/dclm-baseline/toktxt/qwen3.5")
    t.sequence_length = 2048
    t.micro_batch_size = 1
    t.global_batch_size = 1024
    t.max_steps = 4096
    t.optimizer = make_muon_optimizer
    t.lr = 0.0003
    t.scheduler = partial(make_wsd_scheduler, start_lr=1e-05, warmup_ratio=0.03, final_lr=1e-05)
    t.moe_load_balance_type = "global-batch"
    t.moe_load_balance_coef = 0.001
    t.fp8 = False
    t.save_interval = 256
    t.save_location = Path("workspace/checkpoints/qwen3.5-35b-a3b")
    return cfg


if __name__ == "__main__":
    launch(make_cfg())
