"""The reference's public names resolve through the ``pithtrain`` alias package and keep their call signatures
(the list is the reference's public surface: config.py, modules/*, dualpipe/__init__.py, models/*, operators/*,
tasks/*)."""
import importlib
import inspect

import pytest
import torch

from utilities import launch

SURFACE = {
    "pithtrain.config": ["SlottedDefault"],
    "pithtrain.modules.distributed": ["DistributedCfg", "setup_distributed"],
    "pithtrain.modules.training": ["TrainingCfg", "setup_training", "setup_model", "apply_fsdp", "init_weights", "is_muon_param",
                                   "make_muon_optimizer", "make_adamw_optimizer", "make_wsd_scheduler", "make_constant_scheduler"],
    "pithtrain.modules.logging": ["LoggingCfg", "LoggingWandbCfg", "setup_logging", "activate_wandb"],
    "pithtrain.modules.optimizer": ["Muon", "zeropower_via_newtonschulz5", "muon_scale_factor", "orthogonalized_updates"],
    "pithtrain.modules.load_balance": ["make_load_balance_loss_fn", "MoELoadBalanceLossInjector", "MoELoadBalanceLossTracker",
                                       "force_balance"],
    "pithtrain.modules.checkpoint": ["to_canonical_model", "to_canonical_optim", "to_localized_model", "to_localized_optim"],
    "pithtrain.modules.dataset": ["MemmapDataset", "ConcatDataset"],
    "pithtrain.dualpipe": ["DualPipeV", "FP8WeightCacheControl", "WeightGradStore", "set_p2p_tensor_shapes", "set_p2p_tensor_dtype"],
    "pithtrain.dualpipe.dualpipev": ["layer_partition"],
    "pithtrain.models.interface": ["AllToAllSplits", "RoutingInfo", "LayerProtocol", "ModelProtocol"],
    "pithtrain.models.deepseek_v2": ["DeepSeekV2Model"],
    "pithtrain.models.qwen3_moe": ["Qwen3MoeModel"],
    "pithtrain.models.gpt_oss": ["GptOssModel"],
    "pithtrain.models.qwen35_moe": ["Qwen35MoeModel"],
    "pithtrain.tasks.pretrain_lm": ["PretrainLMCfg", "launch", "train_step", "save_checkpoint", "load_checkpoint", "criterion",
                                    "clip_grad_norm_"],
    "pithtrain.tasks.tokenize_corpus": ["TokenizeCorpusCfg", "launch"],
    "pithtrain.tasks.convert_checkpoint": ["ConvertCheckpointCfg", "hf2dcp", "dcp2hf", "launch"],
    "pithtrain.operators.silu_mul": ["silu_mul"],
    "pithtrain.operators.clamped_swiglu": ["clamped_swiglu"],
    "pithtrain.operators.indexed_bias_add": ["indexed_bias_add"],
    "pithtrain.operators.cross_entropy": ["cross_entropy"],
    "pithtrain.operators.flash_attn_v4": ["flash_attn_func", "flash_attn_varlen_func"],
    "pithtrain.operators.gated_delta_rule": ["gated_delta_rule"],
    "pithtrain.operators.ring_attention": ["ring_attention_func", "mla_ring_attention_func"],
    "pithtrain.operators.linear": ["FP8Linear"],
    "pithtrain.operators.grouped_linear": ["GroupedLinear", "FP8GroupedLinear"],
    "pithtrain.operators.all_to_all": ["direct_all_to_all"],
    "pithtrain.operators.token_scatter": ["scatter_for_grouped_gemm", "padded_index_gather", "get_pinned_buffer"],
    "pithtrain.operators.deepgemm_quantize": ["fp8cast_rowwise_colwise", "fp8cast_rowwise_kmajor", "fp8cast_rowwise_transpose",
                                              "fp8cast_rowwise_blockwise_transpose", "fp8cast_blockwise_transpose",
                                              "fp8cast_blockwise_transpose_batched"],
}


@pytest.mark.parametrize("module", sorted(SURFACE))
def test_names_resolve(module):
    m = importlib.import_module(module)
    missing = [n for n in SURFACE[module] if not hasattr(m, n)]
    assert not missing, (module, missing)


def _params(fn):
    return list(inspect.signature(fn).parameters)


def test_signatures():
    from pithtrain.dualpipe.dualpipev import layer_partition
    from pithtrain.modules.dataset import ConcatDataset, MemmapDataset
    from pithtrain.modules.optimizer import Muon
    from pithtrain.modules.training import make_wsd_scheduler
    from pithtrain.operators.flash_attn_v4 import flash_attn_func, flash_attn_varlen_func
    from pithtrain.operators.indexed_bias_add import indexed_bias_add
    from pithtrain.tasks.convert_checkpoint import ConvertCheckpointCfg
    from pithtrain.tasks.tokenize_corpus import TokenizeCorpusCfg

    sig = inspect.signature(make_wsd_scheduler).parameters
    assert [sig[n].default for n in ("start_lr", "warmup_ratio", "final_lr", "decay_ratio", "decay_shape")] == [0.0, 0.0, 0.0, 0.1, "cosine"]
    sig = inspect.signature(Muon.__init__).parameters
    assert (sig["lr"].default, sig["momentum"].default, sig["weight_decay"].default) == (0.02, 0.95, 0.1)
    assert _params(MemmapDataset.__init__)[1:3] == ["path", "sequence_length"] and _params(ConcatDataset.__init__)[2] == "seed"
    assert _params(layer_partition) == ["num_layers", "stage_count", "stage_index"]
    assert _params(flash_attn_func)[:4] == ["q", "k", "v", "softmax_scale"]
    assert _params(flash_attn_varlen_func)[:6] == ["q", "k", "v", "cu_seqlens", "max_seqlen", "softmax_scale"]
    assert _params(indexed_bias_add) == ["x", "bias", "group_ids", "grouped_mm_offs"]
    assert {"tokenizer_name", "source_path", "output_path", "num_workers"} <= set(TokenizeCorpusCfg.__slots__)
    assert {"operation", "load_path", "save_path", "max_shard_size"} <= set(ConvertCheckpointCfg.__slots__)
    assert layer_partition(27, 4, 0) == range(0, 7)


def test_reference_named_operator_helpers():
    from pithtrain.operators.flash_attn_v4 import flash_attn_func, flash_attn_varlen_func
    from pithtrain.operators.indexed_bias_add import indexed_bias_add
    from pithtrain.operators.token_scatter import padded_index_gather, scatter_for_grouped_gemm
    from pithtrain_b200.ops.attention import attention_ref

    torch.manual_seed(0)
    # scatter: groups padded to the alignment, input order kept inside a group, exact allocation
    x = torch.randn(11, 6, requires_grad=True)
    e = torch.tensor([2, 0, 2, 1, 0, 2, 2, 1, 0, 0, 3])
    out, rev, offs, ks, ks_t = scatter_for_grouped_gemm(x, e, 5, padding_alignment=4)
    assert ks == [4, 4, 4, 4, 0] and offs.tolist() == [4, 8, 12, 16, 16] and out.shape == (16, 6) and ks_t.tolist() == ks
    assert torch.equal(out[rev], x.detach())
    for g in range(5):
        rows = rev[e == g]
        lo = 0 if g == 0 else int(offs[g - 1])
        assert rows.tolist() == list(range(lo, lo + rows.numel()))
    pad = torch.ones(16, dtype=torch.bool)
    pad[rev] = False
    assert float(out[pad].abs().max()) == 0.0
    go = torch.randn(16, 6)
    out.backward(go)
    assert torch.equal(x.grad, go[rev])
    # gather without saving the input
    src = torch.randn(7, 3, requires_grad=True)
    idx = torch.tensor([6, 0, 0, 3])
    g = padded_index_gather(src, idx, pad_to_multiple=8)
    assert g.shape == (4, 3) and torch.equal(g, src.detach()[idx])
    g.sum().backward()
    assert src.grad[:, 0].tolist() == [2.0, 0.0, 0.0, 1.0, 0.0, 0.0, 1.0]
    # bias add with cumulative end offsets
    rows = torch.randn(12, 5)
    bias = torch.nn.Parameter(torch.randn(3, 5))
    gid = torch.tensor([0] * 4 + [1] * 0 + [2] * 8)
    y = indexed_bias_add(rows, bias, gid, torch.tensor([4, 4, 12], dtype=torch.int32))
    assert torch.allclose(y, rows + bias.detach()[gid])
    # attention wrappers
    q, k, v = torch.randn(1, 16, 4, 8), torch.randn(1, 16, 2, 8), torch.randn(1, 16, 2, 8)
    assert torch.allclose(flash_attn_func(q, k, v, 0.3, causal=True), attention_ref(q, k, v, True, 0.3), atol=1e-5)
    cu = torch.tensor([0, 5, 16], dtype=torch.int32)
    packed = flash_attn_varlen_func(q[0], k[0], v[0], cu, 11, 0.3, causal=True)
    assert torch.allclose(packed, attention_ref(q, k, v, True, 0.3, cu_seqlens=cu)[0], atol=1e-5)


def test_direct_all_to_all_on_gloo_ranks():
    import compat_worker

    launch(3, compat_worker.run_all_to_all)
