"""The tiny CPU configuration: one forward + cross-entropy backward + AdamW step of a 2-layer Qwen3-MoE-style decoder.

    python benchmarks/pretraining/tiny_cpu.py [--steps 20] [--warmup 3]

Model: 2 layers, hidden 256, 4 query / 2 KV heads of dim 64, RMSNorm eps 1e-6, RoPE theta 1e6, 8 routed experts with a
top-2 softmax router, SwiGLU expert FFN 128, vocab 1024. Batch 2 x 128 token ids drawn uniformly from seed 0, weights
N(0, 0.02), fp32, AdamW lr 3e-4, single process (gloo world size 1). The step goes through the public task API
(``setup_training`` + ``train_step``), i.e. the same engine as the GPU runs with the PyTorch form of every operator.
Prints one JSON line with the median step time; ``tests/test_train_mesh_cpu.py::test_tiny_cpu_configuration_one_step``
checks the same step against a whole-model ``torch.optim.AdamW`` restatement.
"""

import argparse
import json
import os
import statistics
import sys
import time
from functools import partial
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parents[2]))

MODEL = dict(model_type="qwen3_moe", num_hidden_layers=2, hidden_size=256, num_attention_heads=4, num_key_value_heads=2,
             head_dim=64, rms_norm_eps=1e-6, rope_theta=1e6, num_experts=8, num_experts_per_tok=2,
             moe_intermediate_size=128, norm_topk_prob=True, vocab_size=1024, max_position_embeddings=128,
             attention_bias=False)


def main() -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    a = ap.parse_args()
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29531")
    os.environ.setdefault("RANK", "0")
    os.environ.setdefault("WORLD_SIZE", "1")
    os.environ.setdefault("LOCAL_RANK", "0")
    os.environ["CUDA_VISIBLE_DEVICES"] = ""  # this configuration is defined on the CPU

    from pithtrain_b200.modules.distributed import setup_distributed
    from pithtrain_b200.modules.logging import setup_logging
    from pithtrain_b200.modules.training import make_adamw_optimizer, make_constant_scheduler, setup_training
    from pithtrain_b200.tasks.pretrain_lm import PretrainLMCfg, train_step

    cfg = PretrainLMCfg()
    t = cfg.training
    t.model, t.dataset, t.seed = dict(MODEL), None, 0
    t.sequence_length, t.micro_batch_size, t.global_batch_size = 128, 1, 2
    t.lr, t.max_steps, t.moe_load_balance_coef = 3e-4, a.steps + a.warmup, 0.0
    t.optimizer, t.scheduler = partial(make_adamw_optimizer, weight_decay=0.01), make_constant_scheduler
    t.param_dtype, t.grad_dtype = "fp32", "fp32"
    setup_logging(cfg)
    setup_distributed(cfg, failfast=False)
    setup_training(cfg)
    times, loss = [], None
    for i in range(a.steps + a.warmup):
        t0 = time.perf_counter()
        loss = train_step(cfg)["loss"]
        if i >= a.warmup:
            times.append((time.perf_counter() - t0) * 1e3)
    ms = statistics.median(times)
    print(json.dumps({"metric": "step time, tiny Qwen3-MoE decoder on CPU (fwd + CE bwd + AdamW)", "value": ms, "unit": "ms",
                      "higher_is_better": False, "steps": a.steps, "warmup": a.warmup, "dtype": "fp32",
                      "tokens_per_second": 2 * 128 / (ms / 1e3), "final_loss": loss,
                      "config": {"model": MODEL, "batch": "2 x 128", "optimizer": "AdamW lr 3e-4", "device": "cpu"}}))
    return 0


if __name__ == "__main__":
    sys.exit(main())
