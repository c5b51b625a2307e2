"""Worker of the DualPipeV integration test: distributed step vs single-device reference_forward.

Protocol (that of the reference's tests/test_dualpipev.py): every rank builds the whole model from
one seed and runs ``reference_forward`` over all micro-batches; then the same weights are sliced by
pipeline stage and by expert rank, run through ``DualPipeV.step`` on the (pp, ep) mesh, and the
loss and every parameter gradient are compared.
"""

from __future__ import annotations

from types import SimpleNamespace

import torch
import torch.distributed as dist

CONFIGS = {
    "qwen3": dict(model_type="qwen3_moe", hidden_size=64, num_attention_heads=4, num_key_value_heads=2, head_dim=16,
                  rms_norm_eps=1e-6, num_experts=8, num_experts_per_tok=2, moe_intermediate_size=32,
                  norm_topk_prob=True, vocab_size=96, num_hidden_layers=4, max_position_embeddings=64, rope_theta=1e6,
                  attention_bias=False),
    "qwen3_gpu": dict(model_type="qwen3_moe", hidden_size=256, num_attention_heads=4, num_key_value_heads=2, head_dim=64,
                      rms_norm_eps=1e-6, num_experts=8, num_experts_per_tok=2, moe_intermediate_size=128,
                      norm_topk_prob=True, vocab_size=512, num_hidden_layers=4, max_position_embeddings=128,
                      rope_theta=1e6, attention_bias=False),
    "deepseek": dict(model_type="deepseek_v2", hidden_size=64, num_attention_heads=4, qk_rope_head_dim=8,
                     qk_nope_head_dim=16, kv_lora_rank=32, v_head_dim=16, q_lora_rank=None, rms_norm_eps=1e-6,
                     n_routed_experts=8, num_experts_per_tok=2, moe_intermediate_size=32, n_shared_experts=2,
                     first_k_dense_replace=1, intermediate_size=96, routed_scaling_factor=1.0, topk_method="greedy",
                     n_group=1, topk_group=1, vocab_size=96, num_hidden_layers=4, max_position_embeddings=64,
                     rope_theta=10000.0, rope_scaling=None),
    "qwen35": dict(model_type="qwen3_5_moe_text", hidden_size=64, num_attention_heads=4, num_key_value_heads=2, head_dim=16,
                   attn_output_gate=True, layer_types=["linear_attention", "full_attention"] * 2, linear_conv_kernel_dim=4,
                   linear_key_head_dim=8, linear_value_head_dim=8, linear_num_key_heads=2, linear_num_value_heads=4,
                   num_experts=8, num_experts_per_tok=2, moe_intermediate_size=32, shared_expert_intermediate_size=32,
                   rope_parameters=dict(rope_type="default", rope_theta=1e6, partial_rotary_factor=0.5), rms_norm_eps=1e-6,
                   attention_bias=False, vocab_size=96, num_hidden_layers=4, max_position_embeddings=64),
    "gpt_oss": dict(model_type="gpt_oss", hidden_size=64, num_attention_heads=4, num_key_value_heads=2, head_dim=16,
                    rms_norm_eps=1e-5, num_local_experts=8, num_experts_per_tok=2, intermediate_size=32,
                    swiglu_limit=7.0, sliding_window=4, attention_bias=True,
                    layer_types=["sliding_attention", "full_attention"] * 2, vocab_size=96, num_hidden_layers=4,
                    max_position_embeddings=64, initial_context_length=16,
                    rope_scaling=dict(rope_type="yarn", factor=32.0, beta_fast=32.0, beta_slow=1.0, truncate=False,
                                      rope_theta=150000.0)),
}


def _canonical(name: str) -> str:
    return name


def run(rank: int, world: int, model_key: str, pp: int, ep: int, num_chunks: int, overlap: bool = True,
        device_type: str = "cpu", ep_backend: str = "nccl", packed: bool = False, forward_only: bool = False):
    """``packed``: every micro-batch holds two documents (cu_seqlens), attention must not cross the boundary.
    ``forward_only``: ``step`` under ``no_grad`` with ``return_outputs`` (the inference path) against the oracle."""
    from pithtrain_b200.contexts import distributed
    from pithtrain_b200.dualpipe.dualpipev import DualPipeV
    from pithtrain_b200.dualpipe.comm import set_p2p_tensor_dtype, set_p2p_tensor_shapes
    from pithtrain_b200.models import MODEL_CLASSES
    from pithtrain_b200.modules.distributed import DistributedCfg, setup_distributed
    from pithtrain_b200.parallel import ep as ep_mod

    cfg = SimpleNamespace(distributed=DistributedCfg())
    cfg.distributed.pipeline_parallel_size, cfg.distributed.expert_parallel_size = pp, ep
    setup_distributed(cfg, failfast=False)
    dev = distributed.device
    mc = SimpleNamespace(**CONFIGS[model_key])
    Model = MODEL_CLASSES[mc.model_type]
    V, S, B = mc.vocab_size, (16 if device_type == "cpu" else 128), 1
    dtype = torch.float32 if device_type == "cpu" else torch.bfloat16
    dp_like = ep  # every ep rank reads its own micro-batches

    torch.manual_seed(1234)
    ids = torch.randint(0, V, (num_chunks * dp_like * B, S))
    labels = torch.randint(0, V, (num_chunks * dp_like * B, S))

    # ---- reference: whole model on one device, all experts local
    ep_saved = (distributed.ep_size, distributed.ep_rank, distributed.pp_size, distributed.pp_rank)
    distributed.ep_size, distributed.ep_rank, distributed.pp_size, distributed.pp_rank = 1, 0, 1, 0
    ep_mod.set_current(None)
    torch.manual_seed(7)
    prev = torch.get_default_dtype()
    torch.set_default_dtype(dtype)
    with torch.device(dev):
        full = Model(mc, -1)
    torch.set_default_dtype(prev)
    with torch.no_grad():
        for n, p in full.named_parameters():
            if p.dim() >= 2:
                p.normal_(0, 0.05)
            elif "bias" in n or "sinks" in n:
                p.normal_(0, 0.05)
    ref_loss = 0.0
    cuts = [torch.tensor([0, 3 + (i % 5), S], dtype=torch.int32, device=dev) for i in range(ids.shape[0])] if packed else None
    ref_logits = []
    for i in range(ids.shape[0]):
        logits = full.reference_forward(ids[i:i + 1].to(dev), cuts[i] if packed else None)
        ref_logits.append(logits.detach().float().cpu())
        loss = torch.nn.functional.cross_entropy(logits.view(-1, V).float(), labels[i].to(dev), reduction="sum")
        loss.backward()
        ref_loss += float(loss)
    ref_grads = {n: p.grad.detach().float().cpu() for n, p in full.named_parameters()}
    ref_params = {n: p.detach().clone() for n, p in full.named_parameters()}
    del full

    # ---- distributed: slice by stage and expert rank
    distributed.ep_size, distributed.ep_rank, distributed.pp_size, distributed.pp_rank = ep_saved
    ep_mod.setup_exchange(ep_backend)
    torch.set_default_dtype(dtype)
    with torch.device(dev):
        chunks = [Model(mc, 0), Model(mc, 1)]
    torch.set_default_dtype(prev)
    E = getattr(mc, "num_experts", None) or getattr(mc, "n_routed_experts", None) or mc.num_local_experts
    epr = E // ep
    lo, hi = distributed.ep_rank * epr, (distributed.ep_rank + 1) * epr
    with torch.no_grad():
        for m in chunks:
            for n, p in m.named_parameters():
                src = ref_params[n]
                if ".experts." in n:
                    src = src[lo:hi]
                p.copy_(src.to(p.dtype))
    model = DualPipeV(chunks)
    model.overlap = overlap
    set_p2p_tensor_shapes([(B, S, mc.hidden_size)])
    set_p2p_tensor_dtype(dtype)

    def criterion(out, tgt):
        return torch.nn.functional.cross_entropy(out.view(-1, V).float(), tgt.reshape(-1), reduction="sum")

    mine = slice(distributed.ep_rank, None, dp_like)
    my_ids, my_labels = ids[mine].to(dev), labels[mine].to(dev)
    my_cuts = cuts[distributed.ep_rank::dp_like] if packed else None
    if forward_only:
        with torch.no_grad():
            _, outs = model.step(my_ids if distributed.pp_rank == 0 else None, num_chunks=num_chunks,
                                 cu_seqlens=my_cuts if distributed.pp_rank == 0 else None, return_outputs=True)
        if distributed.pp_rank == 0:
            want = torch.cat(ref_logits[distributed.ep_rank::dp_like], 0)
            from utilities import calc_diff

            assert outs.shape == want.shape, (outs.shape, want.shape)
            assert calc_diff(outs.float().cpu(), want) < (1e-6 if dtype == torch.float32 else 1e-3)
        else:
            assert outs is None
        return
    loss, _ = model.step(my_ids if distributed.pp_rank == 0 else None, num_chunks=num_chunks, criterion=criterion,
                         labels=my_labels if distributed.pp_rank == 0 else None,
                         cu_seqlens=my_cuts if distributed.pp_rank == 0 else None)
    total = torch.zeros((), device=dev)
    if loss is not None:
        total += loss.sum()
    dist.all_reduce(total)
    assert abs(float(total) - ref_loss) / ref_loss < (1e-4 if dtype == torch.float32 else 5e-3), (float(total), ref_loss)

    from utilities import calc_diff

    tol = 1e-5 if dtype == torch.float32 else 2e-2
    checked = 0
    for m in chunks:
        for n, p in m.named_parameters():
            g = p.grad
            assert g is not None, f"no grad for {n}"
            g = g.detach().float()
            ref = ref_grads[n]
            if ".experts." in n:
                ref = ref[lo:hi]
            else:
                if ep > 1:
                    dist.all_reduce(g, group=distributed.ep_group)
            d = calc_diff(g.cpu(), ref)
            assert d < tol, f"grad mismatch {n}: calc_diff {d}"
            checked += 1
    assert checked > 0
