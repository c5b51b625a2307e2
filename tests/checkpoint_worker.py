"""Worker for the checkpoint round-trip test: train, save at one (pp, ep) layout, load at another."""
from __future__ import annotations

import sys
from functools import partial
from pathlib import Path

import torch
import torch.distributed as dist

MODEL = dict(model_type="qwen3_moe", hidden_size=32, num_attention_heads=2, num_key_value_heads=1, head_dim=16,
             rms_norm_eps=1e-6, num_experts=4, num_experts_per_tok=2, moe_intermediate_size=16, norm_topk_prob=True,
             vocab_size=64, num_hidden_layers=4, max_position_embeddings=32, rope_theta=1e4, attention_bias=False)


def model_config(key):
    if key == "qwen3":
        return dict(MODEL)
    from dualpipev_worker import CONFIGS

    return dict(CONFIGS[key])


def make_cfg(pp, ep, save_location, steps, model="qwen3"):
    from pithtrain_b200.modules.training import make_muon_optimizer, make_wsd_scheduler
    from pithtrain_b200.tasks.pretrain_lm import PretrainLMCfg

    cfg = PretrainLMCfg()
    cfg.distributed.pipeline_parallel_size, cfg.distributed.expert_parallel_size = pp, ep
    t = cfg.training
    t.model, t.sequence_length, t.lr, t.max_steps = model_config(model), 16, 1e-2, steps
    t.micro_batch_size, t.global_batch_size = 1, 4 * ep
    t.optimizer, t.scheduler = make_muon_optimizer, partial(make_wsd_scheduler, warmup_ratio=0.5)
    t.param_dtype, t.save_location = "fp32", Path(save_location)
    return cfg


def full_state(model):
    """Canonical {fqn: tensor} of everything this rank holds."""
    from pithtrain_b200.modules.checkpoint import to_canonical_model

    return {k: v.detach().clone() for k, v in to_canonical_model(dict(model.state_dict()), model).items()}


def run(rank, world, pp, ep, save_location, phase, model="qwen3", reshard=False):
    from pithtrain_b200.contexts import training
    from pithtrain_b200.modules.checkpoint import load_training_checkpoint, save_training_checkpoint, to_canonical_optim
    from pithtrain_b200.modules.distributed import setup_distributed
    from pithtrain_b200.modules.logging import setup_logging
    from pithtrain_b200.modules.training import setup_training
    from pithtrain_b200.tasks.pretrain_lm import train_step

    cfg = make_cfg(pp, ep, save_location, 4, model)
    cfg.distributed.reshard_params = bool(reshard)
    setup_logging(cfg)
    setup_distributed(cfg, failfast=False)
    setup_training(cfg)
    if phase == "save":
        for _ in range(2):
            train_step(cfg)
        save_training_checkpoint(cfg)
        from pithtrain_b200.contexts import distributed as d
        from pithtrain_b200.modules.checkpoint import build_save_state

        staged = build_save_state(training.model, training.optimizers, training.schedulers)["app"]["model"]
        if d.dp_rank > 0:
            assert not staged, "a data-parallel replica staged model tensors"
        elif d.ep_rank > 0:
            assert staged and all(".experts." in k for k in staged), "a dense tensor was staged by more than one rank"
        st = full_state(training.model)
        opt = to_canonical_optim(training.optimizers, training.model)["state"]
        torch.save({"model": st, "optim": {k: {f: (v.clone() if torch.is_tensor(v) else v) for f, v in e.items()} for k, e in opt.items()}},
                   Path(save_location, f"expect-{rank}.pt"))
    else:
        load_training_checkpoint(cfg)
        assert training.step == 2
        st = full_state(training.model)
        opt = to_canonical_optim(training.optimizers, training.model)["state"]
        expect_m, expect_o = {}, {}
        for f in Path(save_location).glob("expect-*.pt"):
            e = torch.load(f, weights_only=False)
            expect_m.update(e["model"])
            expect_o.update(e["optim"])
        for k, v in st.items():
            assert torch.equal(v, expect_m[k]), f"model mismatch {k}"
        assert opt, "no optimizer state restored"
        for k, e in opt.items():
            for f, v in e.items():
                if torch.is_tensor(v):
                    assert torch.allclose(v.float().cpu(), expect_o[k][f].float().cpu()), f"optimizer mismatch {k}.{f}"
        assert abs(training.schedulers[0].get_last_lr()[0] - 1e-2) < 1e-9
        train_step(cfg)  # resumed run keeps training


def run_strict(rank, world, save_location):
    """A checkpoint with one expert tensor missing: the default load refuses it, ``strict=False`` loads the rest."""
    import torch.distributed.checkpoint as dcp

    from pithtrain_b200.contexts import training
    from pithtrain_b200.modules.checkpoint import build_save_state, load_into
    from pithtrain_b200.modules.distributed import setup_distributed
    from pithtrain_b200.modules.logging import setup_logging
    from pithtrain_b200.modules.training import setup_training

    cfg = make_cfg(1, 1, save_location, 4)
    setup_logging(cfg)
    setup_distributed(cfg, failfast=False)
    setup_training(cfg)
    state = build_save_state(training.model, training.optimizers, training.schedulers)
    victim = next(k for k in state["app"]["model"] if ".experts.3." in k)
    del state["app"]["model"][victim]
    path = Path(save_location, "damaged")
    dcp.save(state, checkpoint_id=str(path))
    try:
        load_into(path, training.model, training.optimizers, training.schedulers)
    except KeyError as e:
        assert victim in str(e), str(e)
    else:
        raise AssertionError("a checkpoint lacking a model tensor loaded without an error")
    load_into(path, training.model, training.optimizers, training.schedulers, strict=False)
