"""HF <-> DCP conversion: generic path, GPT-OSS (MXFP4 + stacked experts), Qwen3.5 (re-nesting)."""
import json

import torch
from safetensors.torch import save_file

from pithtrain_b200.tasks.convert_checkpoint import ConvertCheckpointCfg, dcp2hf, hf2dcp
from pithtrain_b200.tasks.convert_checkpoint._core import read_canonical_model, read_safetensors_dir
from pithtrain_b200.tasks.convert_checkpoint.gpt_oss import FP4_VALUES, dequant_mxfp4


def _cfg(op, src, dst, shard=8 * 1024 ** 3):
    c = ConvertCheckpointCfg()
    c.operation, c.load_path, c.save_path, c.max_shard_size = op, src, dst, shard
    return c


def _write_hf(path, tensors, model_type):
    path.mkdir(parents=True)
    save_file(tensors, str(path / "model.safetensors"))
    json.dump({"model_type": model_type}, open(path / "config.json", "w"))


def test_mxfp4_dequant_lut():
    blocks = torch.tensor([[[0x10 | 0x02, 0xF7] + [0] * 14]], dtype=torch.uint8)  # nibbles: 2,1 | 7,15
    scales = torch.tensor([[128]], dtype=torch.uint8)  # 2^1
    out = dequant_mxfp4(blocks, scales, torch.float32)
    assert out.shape == (1, 32)
    assert out[0, :4].tolist() == [FP4_VALUES[2] * 2, FP4_VALUES[1] * 2, FP4_VALUES[7] * 2, FP4_VALUES[15] * 2]


def test_generic_roundtrip(tmp_path):
    t = {"model.embed_tokens.weight": torch.randn(8, 4), "lm_head.weight": torch.randn(8, 4),
         "model.layers.0.mlp.experts.1.gate_proj.weight": torch.randn(3, 4)}
    _write_hf(tmp_path / "hf", t, "qwen3_moe")
    hf2dcp(_cfg("hf2dcp", tmp_path / "hf", tmp_path / "dcp"))
    canon = read_canonical_model(tmp_path / "dcp")
    assert set(canon) == {"embed_tokens.weight", "lm_head.weight", "layers.0.mlp.experts.1.gate_proj.weight"}
    dcp2hf(_cfg("dcp2hf", tmp_path / "dcp", tmp_path / "out", shard=64))
    back = read_safetensors_dir(tmp_path / "out")
    assert set(back) == set(t) and all(torch.equal(back[k], t[k]) for k in t)
    index = json.load(open(tmp_path / "out" / "model.safetensors.index.json"))
    assert len(set(index["weight_map"].values())) > 1  # sharded by max_shard_size


def test_gpt_oss_roundtrip(tmp_path):
    E, I, H = 2, 4, 32
    t = {"model.layers.0.mlp.experts.gate_up_proj": torch.randn(E, H, 2 * I).bfloat16(),
         "model.layers.0.mlp.experts.gate_up_proj_bias": torch.randn(E, 2 * I).bfloat16(),
         "model.layers.0.mlp.experts.down_proj": torch.randn(E, I, H).bfloat16(),
         "model.layers.0.mlp.experts.down_proj_bias": torch.randn(E, H).bfloat16(),
         "model.layers.0.mlp.router.weight": torch.randn(E, H).bfloat16()}
    _write_hf(tmp_path / "hf", t, "gpt_oss")
    hf2dcp(_cfg("hf2dcp", tmp_path / "hf", tmp_path / "dcp"))
    canon = read_canonical_model(tmp_path / "dcp")
    assert canon["layers.0.mlp.experts.1.gate_up_proj"].shape == (2 * I, H)  # [out, in]
    assert torch.equal(canon["layers.0.mlp.experts.1.gate_up_proj"], t["model.layers.0.mlp.experts.gate_up_proj"][1].t())
    dcp2hf(_cfg("dcp2hf", tmp_path / "dcp", tmp_path / "out"))
    back = read_safetensors_dir(tmp_path / "out")
    assert set(back) == set(t) and all(torch.equal(back[k], t[k]) for k in t)


def test_gpt_oss_mxfp4_import(tmp_path):
    E, O, G = 2, 6, 2
    blocks = torch.randint(0, 256, (E, O, G, 16), dtype=torch.uint8)
    scales = torch.randint(120, 134, (E, O, G), dtype=torch.uint8)
    t = {"model.layers.0.mlp.experts.down_proj_blocks": blocks, "model.layers.0.mlp.experts.down_proj_scales": scales}
    _write_hf(tmp_path / "hf", t, "gpt_oss")
    hf2dcp(_cfg("hf2dcp", tmp_path / "hf", tmp_path / "dcp"))
    canon = read_canonical_model(tmp_path / "dcp")
    ref = dequant_mxfp4(blocks, scales)
    assert torch.equal(canon["layers.0.mlp.experts.0.down_proj"], ref[0])


def test_qwen35_roundtrip(tmp_path):
    E, I, H = 2, 3, 4
    t = {"model.language_model.layers.0.mlp.experts.gate_up_proj": torch.randn(E, 2 * I, H),
         "model.language_model.layers.0.mlp.experts.down_proj": torch.randn(E, H, I),
         "model.language_model.layers.0.linear_attn.A_log": torch.randn(4),
         "model.visual.patch_embed.weight": torch.randn(2, 2), "mtp.fc.weight": torch.randn(2, 2),
         "lm_head.weight": torch.randn(8, H)}
    _write_hf(tmp_path / "hf", t, "qwen3_5_moe")
    hf2dcp(_cfg("hf2dcp", tmp_path / "hf", tmp_path / "dcp"))
    canon = read_canonical_model(tmp_path / "dcp")
    assert "layers.0.mlp.experts.1.gate_up_proj.weight" in canon and not any("visual" in k or "mtp" in k for k in canon)
    dcp2hf(_cfg("dcp2hf", tmp_path / "dcp", tmp_path / "out"))
    back = read_safetensors_dir(tmp_path / "out")
    kept = {k: v for k, v in t.items() if not k.startswith(("model.visual.", "mtp."))}
    assert set(back) == set(kept) and all(torch.equal(back[k], kept[k]) for k in kept)
