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


@pytest.mark.parametrize("save_layout,load_layout", [((1, 1), (1, 1)), ((2, 2), (1, 4)), ((1, 2), (2, 1))])
def test_reshard_roundtrip(tmp_path, save_layout, load_layout):
    (pp0, ep0), (pp1, ep1) = save_layout, load_layout
    launch(pp0 * ep0, checkpoint_worker.run, pp0, ep0, str(tmp_path), "save")
    launch(pp1 * ep1, checkpoint_worker.run, pp1, ep1, str(tmp_path), "load")
