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
    d.sharding_strategy, _, extra = strategy.partition("+")
    d.reshard_params = extra == "reshard"
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
        if d.reshard_params:
            # between steps a rank holds only the parameters it owns: the other owners' regions are freed
            sharded = [g for g in training.shard_groups if g.group_size > 1]
            assert sharded and all(g.reshard_params and not g.params_resident() for g in sharded)
            assert all(g.own_param.numel() * g.group_size == g.flat_param.numel() for g in sharded)
    if rank == 0:
        with open(out_path, "w") as f:
            json.dump(rows, f)


TINY_CPU = dict(model_type="qwen3_moe", num_hidden_layers=2, hidden_size=256, num_attention_heads=4, num_key_value_heads=2,
                head_dim=64, rms_norm_eps=1e-6, rope_theta=1e6, num_experts=8, num_experts_per_tok=2,
                moe_intermediate_size=128, norm_topk_prob=True, vocab_size=1024, max_position_embeddings=128,
                attention_bias=False)


def run_tiny_cpu_step(rank: int, world: int):
    """Tiny Qwen3-MoE decoder (2 layers, hidden 256, 4 query / 2 KV heads of dim 64, 8 experts top-2, FFN 128, vocab
    1024), batch 2 x 128, fp32: one forward + cross-entropy backward + AdamW step (lr 3e-4) through the public task
    API, checked against the whole model on one device with ``torch.optim.AdamW``."""
    from functools import partial
    from types import SimpleNamespace

    import torch

    from pithtrain_b200.contexts import distributed, training
    from pithtrain_b200.models import MODEL_CLASSES
    from pithtrain_b200.modules.checkpoint import strip_prefix
    from pithtrain_b200.modules.distributed import setup_distributed
    from pithtrain_b200.modules.logging import setup_logging
    from pithtrain_b200.modules.training import make_adamw_optimizer, make_constant_scheduler, setup_training
    from pithtrain_b200.tasks.pretrain_lm import PretrainLMCfg, get_global_batch, train_step

    cfg = PretrainLMCfg()
    t = cfg.training
    t.model, t.dataset = dict(TINY_CPU), None
    t.sequence_length, t.micro_batch_size, t.global_batch_size = 128, 1, 2
    t.lr, t.max_steps, t.moe_load_balance_coef = 3e-4, 1, 0.0
    t.optimizer, t.scheduler = partial(make_adamw_optimizer, weight_decay=0.01), make_constant_scheduler
    t.param_dtype, t.grad_dtype = "fp32", "fp32"
    setup_logging(cfg)
    setup_distributed(cfg, failfast=False)
    setup_training(cfg)
    before = {strip_prefix(k): v.detach().clone() for k, v in training.model.state_dict().items()}
    tokens, labels = (x.clone() for x in get_global_batch(cfg, distributed.device))
    assert tokens.shape == (2, 128) and int(tokens.max()) < 1024
    metrics = train_step(cfg)
    after = {strip_prefix(k): v.detach().clone() for k, v in training.model.state_dict().items()}

    full = MODEL_CLASSES["qwen3_moe"](SimpleNamespace(**TINY_CPU), -1)
    missing = full.load_state_dict({k: v for k, v in before.items() if k in full.state_dict()}, strict=False)
    assert not [k for k in missing.missing_keys if "inv_freq" not in k and "cos" not in k and "sin" not in k], missing
    opt = torch.optim.AdamW(full.parameters(), lr=3e-4, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.01)
    loss = 0.0
    for i in range(2):
        logits = full.reference_forward(tokens[i:i + 1])
        loss = loss + torch.nn.functional.cross_entropy(logits.view(-1, 1024).float(), labels[i].long(), reduction="sum")
    loss = loss / labels.numel()
    loss.backward()
    norm = torch.nn.utils.clip_grad_norm_(full.parameters(), t.max_grad_norm)
    opt.step()
    assert abs(float(loss.detach()) - metrics["loss"]) < 1e-5 * float(loss), (float(loss), metrics["loss"])
    assert abs(float(norm) - metrics["gradient_norm"]) < 1e-4 * float(norm), (float(norm), metrics["gradient_norm"])
    want = full.state_dict()
    moved = 0
    for k, v in after.items():
        if k not in want:
            continue
        # the first AdamW step moves an element by lr * g / (|g| + eps): where |g| is of the order of eps the fp32
        # summation order shows, so the bulk is held to 1e-6 and single elements to a fraction of lr
        err = (v - want[k]).abs()
        assert float(err.mean()) < 1e-6 and float(err.max()) < 1e-4, (k, float(err.mean()), float(err.max()))
        moved += int(not torch.equal(v, before[k]))
    assert moved >= 20, moved
    # first moments are 0.1 * gradient: an eps-free comparison of every gradient the step produced
    names = {id(p): strip_prefix(n) for n, p in training.model.named_parameters()}
    grads = {n: p.grad for n, p in full.named_parameters()}
    checked = 0
    for opt_mine in training.optimizers:
        for p, st in opt_mine.state.items():
            n = names[id(p)]
            if n in grads and "exp_avg" in st:
                # the oracle's gradient was clipped in place by clip_grad_norm_ above, like the framework's
                assert torch.allclose(st["exp_avg"], 0.1 * grads[n], atol=1e-9, rtol=2e-3), n
                checked += 1
    assert checked >= 20, checked


def run_memory_trace(rank: int, world: int, out_path: str):
    """Two steps of the tiny model with a memory trace attached: one row per schedule action, forward actions save
    tensors for the backward, and the traced step computes what the untraced one does."""
    import json

    import torch

    from pithtrain_b200.contexts import training
    from pithtrain_b200.dualpipe.schedule import build_schedule
    from pithtrain_b200.modules.distributed import setup_distributed
    from pithtrain_b200.modules.logging import setup_logging
    from pithtrain_b200.modules.training import make_adamw_optimizer, make_constant_scheduler, setup_training
    from pithtrain_b200.tasks.pretrain_lm import PretrainLMCfg, train_step
    from pithtrain_b200.tools.memory_trace import MemoryTrace

    def make():
        cfg = PretrainLMCfg()
        cfg.distributed.pipeline_parallel_size = world
        t = cfg.training
        t.model = dict(TINY_CPU, hidden_size=64, head_dim=16, moe_intermediate_size=32, vocab_size=128, num_hidden_layers=4)
        t.sequence_length, t.micro_batch_size, t.global_batch_size = 32, 1, 4
        t.lr, t.max_steps, t.moe_load_balance_coef, t.dataset = 1e-3, 4, 0.0, None
        t.optimizer, t.scheduler = make_adamw_optimizer, make_constant_scheduler
        t.param_dtype, t.grad_dtype = "fp32", "fp32"
        return cfg

    cfg = make()
    setup_logging(cfg)
    setup_distributed(cfg, failfast=False)
    setup_training(cfg)
    plain = train_step(cfg)["gradient_norm"]
    training.step = 0  # same batch again, now traced
    lines = []
    trace = MemoryTrace(ranks=None, sink=lines.append).attach(training.model)
    # the optimizer already moved the weights once, so compare against a fresh run below instead of `plain`
    traced = train_step(cfg)["gradient_norm"]
    trace.detach()
    acts = build_schedule(world, rank, 4)
    assert [r.action for r in trace.rows] == [repr(a) for a in acts], (trace.rows, acts)
    assert len(lines) == len(acts) and all("saved-by-autograd" in ln for ln in lines)
    saved = {r.action: r.saved_for_backward for r in trace.rows}
    assert all(b > 0 for a, b in saved.items() if a.startswith("F")), saved
    assert all(r.saved_for_backward == 0 for r in trace.rows if r.action == "W")
    assert trace.peak() is not None and torch.isfinite(torch.tensor(traced)) and plain > 0
    if rank == 0:
        json.dump({"rows": len(trace.rows)}, open(out_path, "w"))


def run_with_fake_wandb(rank: int, world: int, out_path: str):
    """Two steps with tracking configured and a stand-in ``wandb`` module: the run is created lazily after the first
    good step, metrics are defined against ``train/step`` and every step logs the trainer's metric set."""
    import json
    import sys
    import types

    calls = {"init": [], "define": [], "log": []}

    class Run:
        def log(self, row):
            calls["log"].append(dict(row))

    fake = types.ModuleType("wandb")
    fake.init = lambda **kw: (calls["init"].append({k: (v if k != "config" else sorted(v)) for k, v in kw.items()}), Run())[1]
    fake.define_metric = lambda name, step_metric=None: calls["define"].append((name, step_metric))
    sys.modules["wandb"] = fake

    from pithtrain_b200.contexts import logging as log_ctx
    from pithtrain_b200.modules.distributed import setup_distributed
    from pithtrain_b200.modules.logging import LoggingWandbCfg, setup_logging
    from pithtrain_b200.modules.training import make_adamw_optimizer, make_constant_scheduler, setup_training
    from pithtrain_b200.tasks.pretrain_lm import PretrainLMCfg, train_step

    cfg = PretrainLMCfg()
    t = cfg.training
    t.model = dict(TINY_CPU, hidden_size=64, head_dim=16, moe_intermediate_size=32, vocab_size=128)
    t.sequence_length, t.micro_batch_size, t.global_batch_size = 16, 1, 2
    t.lr, t.max_steps, t.dataset = 1e-3, 2, None
    t.moe_load_balance_coef, t.moe_load_balance_type = 1e-3, "micro-batch"
    t.optimizer, t.scheduler = make_adamw_optimizer, make_constant_scheduler
    t.param_dtype, t.grad_dtype = "fp32", "fp32"
    w = LoggingWandbCfg()
    w.entity, w.project, w.name, w.group = "team", "proj", "tiny", "ci"
    cfg.logging.wandb = w
    setup_logging(cfg)
    setup_distributed(cfg, failfast=False)
    setup_training(cfg)
    assert log_ctx.wandb is None and not calls["init"]  # nothing is created before a step has succeeded
    train_step(cfg)
    train_step(cfg)
    assert len(calls["init"]) == 1 and calls["init"][0]["entity"] == "team" and calls["init"][0]["name"] == "tiny"
    assert all(step == "train/step" for _, step in calls["define"]) and len(calls["define"]) >= 6
    assert len(calls["log"]) == 2 and [r["train/step"] for r in calls["log"]] == [0, 1]
    keys = set(calls["log"][0])
    assert {"train/cross-entropy-loss", "train/load-balance-loss", "train/learning-rate", "train/gradient-norm",
            "infra/tokens-per-second", "infra/peak-gpu-memory", "infra/step-time"} <= keys
    assert calls["log"][0]["train/load-balance-loss"] > 0
    json.dump(calls["log"], open(out_path, "w"))


def run_app_state_roundtrip(rank: int, world: int):
    """AppState of a trained tiny model loads into a freshly built, perturbed one: parameters, optimizer
    state and scheduler position are equal afterwards and the next step produces the same loss."""
    import copy

    import torch

    from pithtrain_b200.contexts import training
    from pithtrain_b200.modules.distributed import setup_distributed
    from pithtrain_b200.modules.logging import setup_logging
    from pithtrain_b200.modules.training import make_muon_optimizer, make_wsd_scheduler, setup_training
    from pithtrain_b200.tasks.pretrain_lm import AppState, PretrainLMCfg, train_step
    from functools import partial

    def make(seed):
        cfg = PretrainLMCfg()
        t = cfg.training
        t.model = dict(TINY_CPU, hidden_size=64, head_dim=16, moe_intermediate_size=32, vocab_size=128)
        t.sequence_length, t.micro_batch_size, t.global_batch_size = 16, 1, 2
        t.lr, t.max_steps, t.dataset, t.seed = 1e-2, 8, None, seed
        t.optimizer, t.scheduler = make_muon_optimizer, partial(make_wsd_scheduler, warmup_ratio=0.5)
        t.param_dtype, t.grad_dtype = "fp32", "fp32"
        return cfg

    cfg = make(1234)
    setup_logging(cfg)
    setup_distributed(cfg, failfast=False)
    setup_training(cfg)
    train_step(cfg)
    train_step(cfg)
    saved = copy.deepcopy(AppState(training.model, training.optimizers, training.schedulers).state_dict())
    assert set(saved) == {"model", "optimizer", "scheduler"}
    assert all(not k.startswith("module.") for k in saved["model"])
    assert any(".experts.7." in k for k in saved["model"]) and not any(k.endswith("experts.gate_proj.weight") for k in saved["model"])
    assert set(AppState(training.model, model_only=True).state_dict()) == {"model"}
    want = train_step(cfg)["loss"]

    cfg2 = make(1234)  # same seed: the synthetic token stream is a function of it
    setup_training(cfg2)
    with torch.no_grad():
        for p in training.model.parameters():
            p.add_(torch.randn_like(p) * 0.01)  # a different starting point than the saved run had
    fresh = AppState(training.model, training.optimizers, training.schedulers)
    assert any(not torch.equal(v, saved["model"][k]) for k, v in fresh.state_dict()["model"].items())
    fresh.load_state_dict(saved)
    again = fresh.state_dict()
    for k, v in saved["model"].items():
        assert torch.equal(again["model"][k], v), k
    for k, entry in saved["optimizer"]["state"].items():
        for f, v in entry.items():
            if torch.is_tensor(v):
                assert torch.allclose(again["optimizer"]["state"][k][f].float(), v.float()), (k, f)
    assert training.schedulers[0].get_last_lr() == [saved["scheduler"][0]["_last_lr"][0]]
    training.step = 2
    got = train_step(cfg2)["loss"]
    assert abs(got - want) < 1e-5 * abs(want), (got, want)


def run_benchmark_mode(rank: int, world: int, out_path: str):
    """``benchmark=True`` (the reference's throughput protocol): routing is replaced by a round-robin assignment, so
    every expert receives the same number of rows and the load-balance metric is exactly 1."""
    import json
    import math

    from pithtrain_b200.modules.distributed import setup_distributed
    from pithtrain_b200.modules.logging import setup_logging
    from pithtrain_b200.modules.training import make_muon_optimizer, make_constant_scheduler, setup_training
    from pithtrain_b200.tasks.pretrain_lm import PretrainLMCfg, train_step

    cfg = PretrainLMCfg()
    cfg.distributed.expert_parallel_size = world
    t = cfg.training
    t.model = dict(TINY_CPU, hidden_size=64, head_dim=16, moe_intermediate_size=32, vocab_size=128)
    t.sequence_length, t.micro_batch_size, t.global_batch_size = 32, 1, 2 * world
    t.lr, t.max_steps, t.dataset, t.benchmark = 1e-6, 2, None, True
    t.moe_load_balance_type, t.moe_load_balance_coef = "global-batch", 1e-3
    t.optimizer, t.scheduler = make_muon_optimizer, make_constant_scheduler
    t.param_dtype, t.grad_dtype = "fp32", "fp32"
    setup_logging(cfg)
    setup_distributed(cfg, failfast=False)
    setup_training(cfg)
    rows = [train_step(cfg) for _ in range(2)]
    for m in rows:
        assert math.isfinite(m["gradient_norm"]) and abs(m["load_balance_loss"] - 1.0) < 1e-3, m
    if rank == 0:
        assert all(math.isfinite(m["loss"]) for m in rows)
        json.dump([m["load_balance_loss"] for m in rows], open(out_path, "w"))


def run_expert_grad_scaling(rank: int, world: int):
    """``expert_grad_scaling``: the default divides expert gradients by ``ep`` (mesh-invariant loss curves); ``reference``
    keeps the extra factor ``ep`` the reference's per-mesh averaging produces, so the first step's gradient norm is
    larger by exactly the expert share."""
    from pithtrain_b200.contexts import training
    from pithtrain_b200.modules.distributed import setup_distributed
    from pithtrain_b200.modules.logging import setup_logging
    from pithtrain_b200.modules.training import make_adamw_optimizer, make_constant_scheduler, setup_training
    from pithtrain_b200.tasks.pretrain_lm import PretrainLMCfg, train_step

    norms = {}
    for i, mode in enumerate(("global-mean", "reference")):
        cfg = PretrainLMCfg()
        cfg.distributed.expert_parallel_size = world
        t = cfg.training
        t.model = dict(TINY_CPU, hidden_size=64, head_dim=16, moe_intermediate_size=32, vocab_size=128)
        t.sequence_length, t.micro_batch_size, t.global_batch_size = 16, 1, 2 * world
        t.lr, t.max_steps, t.dataset, t.max_grad_norm = 0.0, 1, None, 1e9
        t.optimizer, t.scheduler = make_adamw_optimizer, make_constant_scheduler
        t.param_dtype, t.grad_dtype = "fp32", "fp32"
        t.expert_grad_scaling = mode
        if i == 0:
            setup_logging(cfg)
            setup_distributed(cfg, failfast=False)
        setup_training(cfg)
        divisors = sorted({g.grad_divisor for g in training.shard_groups})
        assert divisors == ([1, world] if mode == "global-mean" else [1]), (mode, divisors)
        norms[mode] = train_step(cfg)["gradient_norm"]
    assert norms["reference"] > norms["global-mean"] * 1.0001, norms
