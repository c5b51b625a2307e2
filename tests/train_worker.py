"""Worker: a few optimizer steps of the tiny Qwen3-MoE through the public task API on a given mesh."""
from __future__ import annotations

import json


def run(rank: int, world: int, pp: int, ep: int, cp: int, strategy: str, out_path: str, optimizer: str = "adamw",
        steps: int = 4, model: str = "qwen3"):
    from pithtrain_b200.contexts import training
    from pithtrain_b200.modules.distributed import setup_distributed
    from pithtrain_b200.modules.logging import setup_logging
    from pithtrain_b200.modules.training import (make_adamw_optimizer, make_constant_scheduler, make_muon_optimizer,
                                                 setup_training)
    from pithtrain_b200.tasks.pretrain_lm import PretrainLMCfg, train_step

    cfg = PretrainLMCfg()
    d = cfg.distributed
    d.pipeline_parallel_size, d.expert_parallel_size, d.context_parallel_size = pp, ep, cp
    d.sharding_strategy = strategy
    t = cfg.training
    t.model = dict(model_type="qwen3_moe", hidden_size=64, num_attention_heads=4, num_key_value_heads=2, head_dim=16,
                   rms_norm_eps=1e-6, num_experts=8, num_experts_per_tok=2, moe_intermediate_size=32,
                   norm_topk_prob=True, vocab_size=128, num_hidden_layers=4, max_position_embeddings=64,
                   rope_theta=1e6, attention_bias=False)
    if model != "qwen3":
        from dualpipev_worker import CONFIGS

        t.model = dict(CONFIGS[model])
    t.sequence_length, t.micro_batch_size, t.global_batch_size = 32, 1, 8
    t.lr, t.max_steps = 2e-3, steps
    t.optimizer = make_muon_optimizer if optimizer == "muon" else make_adamw_optimizer
    t.scheduler = make_constant_scheduler
    t.param_dtype, t.grad_dtype = "fp32", "fp32"
    t.moe_load_balance_coef = 0.0
    t.dataset = None
    setup_logging(cfg)
    setup_distributed(cfg, failfast=False)
    setup_training(cfg)
    rows = []
    for _ in range(steps):
        m = train_step(cfg)
        rows.append({"loss": m.get("loss"), "gradient_norm": m["gradient_norm"]})
    if rank == 0:
        with open(out_path, "w") as f:
            json.dump(rows, f)
