"""Pre-train DeepSeek-V2-Lite: pipeline x2, expert x2, context x1; the data-parallel width is whatever is left."""

from functools import partial
from pathlib import Path

from pithtrain_b200.modules.training import make_muon_optimizer, make_wsd_scheduler
from pithtrain_b200.tasks.pretrain_lm import PretrainLMCfg, launch

HERE = Path(__file__).resolve().parent


def make_cfg() -> PretrainLMCfg:
    cfg = PretrainLMCfg()

    mesh = cfg.distributed
    mesh.pipeline_parallel_size = 2
    mesh.expert_parallel_size = 2
    mesh.context_parallel_size = 1

    t = cfg.training
    t.model = HERE / "config.json"
    t.dataset = Path("workspace/datasets/dclm-baseline/toktxt/deepseek-v2")
    t.sequence_length = 2048
    t.micro_batch_size = 1
    t.global_batch_size = 1024
    t.max_steps = 64
    t.optimizer = make_muon_optimizer
    t.lr = 0.0001
    t.scheduler = partial(make_wsd_scheduler, start_lr=0.0001, warmup_ratio=0.0, final_lr=0.0001)
    t.moe_load_balance_type = "sequence"
    t.moe_load_balance_coef = 0.003
    t.fp8 = False
    t.save_interval = 256
    t.save_location = Path("workspace/checkpoints/deepseek-v2-lite")
    return cfg


if __name__ == "__main__":
    launch(make_cfg())
