"""Checkpoint round trips: canonical key mapping and resharding across (pp, ep) layouts."""
import pytest
import torch

from utilities import launch
import checkpoint_worker


def test_canonical_keys():
    from pithtrain_b200.modules.checkpoint import canonical_expert_keys, is_stacked_expert_key, strip_prefix

    assert strip_prefix("module.1.layers.7.mlp.gate.weight") == "layers.7.mlp.gate.weight"
    assert is_stacked_expert_key("module.0.layers.1.mlp.experts.gate_proj.weight")
    assert not is_stacked_expert_key("layers.1.mlp.experts.3.gate_proj.weight")
    assert not is_stacked_expert_key("layers.1.mlp.shared_experts.gate_proj.weight")
    assert canonical_expert_keys("module.0.layers.1.mlp.experts.gate_up_proj", 2, 3) == [
        "layers.1.mlp.experts.6.gate_up_proj", "layers.1.mlp.experts.7.gate_up_proj"]


@pytest.mark.parametrize("save_layout,load_layout", [((2, 2), (1, 4)), ((1, 2), (2, 1))])
def test_reshard_roundtrip(tmp_path, save_layout, load_layout):
    (pp0, ep0), (pp1, ep1) = save_layout, load_layout
    launch(pp0 * ep0, checkpoint_worker.run, pp0, ep0, str(tmp_path), "save")
    launch(pp1 * ep1, checkpoint_worker.run, pp1, ep1, str(tmp_path), "load")


def test_data_parallel_replicas_stage_nothing(tmp_path):
    """Saved at dp2 x ep2 (only the first replica stages model tensors, dense ones only on its first ep rank), loaded at
    dp1 x ep2: every tensor is there exactly once."""
    launch(4, checkpoint_worker.run, 1, 2, str(tmp_path), "save")
    launch(2, checkpoint_worker.run, 1, 2, str(tmp_path), "load")


def test_checkpoint_with_parameters_sharded_between_steps(tmp_path):
    """``reshard_params``: the save gathers the released parameter regions first, the load fills owned and foreign
    parameters alike, and the resumed job (again with released parameters) keeps training."""
    launch(4, checkpoint_worker.run, 1, 2, str(tmp_path), "save", "qwen3", True)
    launch(4, checkpoint_worker.run, 1, 2, str(tmp_path), "load", "qwen3", True)


@pytest.mark.parametrize("model", ["deepseek", "gpt_oss"])
def test_muon_state_roundtrip_other_families(tmp_path, model):
    """Muon momentum and AdamW moments of the MLA / shared-expert / dense-first-layer model and of the model with
    expert biases survive a save at pp2·ep2 and a load at pp1·ep2 (pithtrain tests/test_muon_checkpoint.py:109-125)."""
    launch(4, checkpoint_worker.run, 2, 2, str(tmp_path), "save", model)
    launch(2, checkpoint_worker.run, 1, 2, str(tmp_path), "load", model)


def test_param_group_membership_survives_canonical_roundtrip():
    """Which optimizer a parameter belongs to, its hyper-parameters and its state survive canonical -> localized, with
    stacked expert parameters fanned out to global expert indices (pithtrain tests/test_muon.py:164-206)."""
    from pithtrain_b200.modules.checkpoint import to_canonical_optim, to_localized_optim
    from pithtrain_b200.modules.optimizer import AdamW, Muon
    from pithtrain_b200.modules.training import is_muon_param

    class Experts(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.gate_proj = torch.nn.Module()
            self.gate_proj.weight = torch.nn.Parameter(torch.randn(2, 6, 8))

    def build():
        torch.manual_seed(0)
        layer = torch.nn.Module()
        layer.self_attn = torch.nn.Module()
        layer.self_attn.q_proj = torch.nn.Linear(8, 8, bias=True)
        layer.input_layernorm = torch.nn.Module()
        layer.input_layernorm.weight = torch.nn.Parameter(torch.ones(8))
        layer.mlp = torch.nn.Module()
        layer.mlp.experts = Experts()
        layer.mlp.gate = torch.nn.Linear(8, 4, bias=False)
        stage = torch.nn.Module()
        stage.layers = torch.nn.ModuleDict({"1": layer})
        model = torch.nn.Module()  # the pipeline wrapper names its stages ``module.<N>``
        model.module = torch.nn.Sequential(stage)
        named = list(model.named_parameters())
        muon = [p for n, p in named if is_muon_param(n, p)]
        rest = [p for n, p in named if not is_muon_param(n, p)]
        return model, (Muon(muon, lr=0.02, momentum=0.9, weight_decay=0.1), AdamW(rest, lr=0.01, weight_decay=0.0))

    model, opts = build()
    for p in model.parameters():
        p.grad = torch.randn_like(p)
    for o in opts:
        o.step()
    canon = to_canonical_optim(opts, model, ep_rank=1)
    groups = {g["type"]: g for g in canon["param_groups"]}
    assert set(groups["Muon"]["params"]) == {"layers.1.self_attn.q_proj.weight", "layers.1.mlp.experts.2.gate_proj.weight",
                                             "layers.1.mlp.experts.3.gate_proj.weight"}
    assert set(groups["AdamW"]["params"]) == {"layers.1.self_attn.q_proj.bias", "layers.1.input_layernorm.weight",
                                              "layers.1.mlp.gate.weight"}
    assert groups["Muon"]["lr"] == 0.02 and groups["AdamW"]["lr"] == 0.01
    stacked = opts[0].state[model.module[0].layers["1"].mlp.experts.gate_proj.weight]
    field = next(k for k, v in stacked.items() if torch.is_tensor(v) and v.shape == (2, 6, 8))
    assert torch.equal(canon["state"]["layers.1.mlp.experts.3.gate_proj.weight"][field], stacked[field][1])

    model2, opts2 = build()
    opts2[0].param_groups[0]["lr"] = 99.0
    to_localized_optim(canon, model2, opts2, ep_rank=1)
    assert opts2[0].param_groups[0]["lr"] == 0.02
    again = to_canonical_optim(opts2, model2, ep_rank=1)
    assert [g["params"] for g in again["param_groups"]] == [g["params"] for g in canon["param_groups"]]
    assert again["state"].keys() == canon["state"].keys()
    for k, entry in canon["state"].items():
        for f, v in entry.items():
            if torch.is_tensor(v):
                assert torch.equal(again["state"][k][f].float(), v.float()), (k, f)


def test_interrupted_save_is_skipped_on_resume(tmp_path):
    """Host-side fault injection: a newer checkpoint directory without ``.metadata`` (what a save killed half-way
    leaves behind) is ignored and the job resumes from the complete checkpoint before it; a complete directory whose
    shard file was truncated makes the resume fail loudly instead of training on from a half-loaded state."""
    from pithtrain_b200.modules.checkpoint import is_complete, latest_checkpoint

    launch(2, checkpoint_worker.run, 1, 2, str(tmp_path), "save")
    good = latest_checkpoint(tmp_path)
    assert good is not None and good.name == "step-00000002" and is_complete(good)
    partial = good.parent / "step-00000003"
    partial.mkdir()
    (partial / "__0_0.distcp").write_bytes(b"half a shard")
    assert latest_checkpoint(tmp_path) == good
    launch(2, checkpoint_worker.run, 1, 2, str(tmp_path), "load")  # asserts that it resumed at step 2

    shard = sorted(good.glob("*.distcp"))[0]
    shard.write_bytes(shard.read_bytes()[:64])
    with pytest.raises(AssertionError, match="failed"):  # every rank exits non-zero; nobody trains on
        launch(2, checkpoint_worker.run, 1, 2, str(tmp_path), "load")


def test_load_refuses_a_checkpoint_that_lacks_model_tensors(tmp_path):
    launch(1, checkpoint_worker.run_strict, str(tmp_path), timeout=300.0)


def test_app_state_roundtrip_in_one_process():
    import train_worker

    launch(1, train_worker.run_app_state_roundtrip, timeout=300.0)
