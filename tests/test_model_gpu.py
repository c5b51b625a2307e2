"""Qwen3-MoE staged execution on the GPU kernels vs the plain-PyTorch reference_forward."""
import pytest
import torch
from types import SimpleNamespace

pytestmark = pytest.mark.gpu


def calc_diff(x, y):
    x, y = x.double(), y.double()
    d = (x * x + y * y).sum()
    return 0.0 if d == 0 else float(1 - 2 * (x * y).sum() / d)


@pytest.mark.parametrize("fp8", [False, True])
def test_qwen3_staged_vs_reference(fp8):
    """``fp8``: forward and input-gradient GEMMs of the projections and experts run block-scaled e4m3 (looser bound)."""
    from pithtrain_b200 import _native
    from pithtrain_b200.ops import fp8_linear

    fp8_linear.enable(fp8)
    try:
        _staged_vs_reference(_native, fp8)
    finally:
        fp8_linear.enable(False)


def _staged_vs_reference(_native, fp8):
    from pithtrain_b200.ops import fp8_linear

    from pithtrain_b200.contexts import distributed
    from pithtrain_b200.dualpipe.execution import ChunkRecord, model_backward, model_forward
    from pithtrain_b200.models.qwen3_moe import Qwen3MoeModel

    distributed.reset_single_process()
    distributed.device = torch.device("cuda", 0)
    torch.manual_seed(0)
    cfg = SimpleNamespace(hidden_size=512, num_attention_heads=8, num_key_value_heads=2, head_dim=128, rms_norm_eps=1e-6,
                          num_experts=16, num_experts_per_tok=4, moe_intermediate_size=256, norm_topk_prob=True,
                          vocab_size=2048, num_hidden_layers=2, max_position_embeddings=256, rope_theta=1e6,
                          attention_bias=False)
    prev = torch.get_default_dtype()
    torch.set_default_dtype(torch.bfloat16)
    try:
        with torch.device("cuda"):
            m = Qwen3MoeModel(cfg, -1)
    finally:
        torch.set_default_dtype(prev)
    ids = torch.randint(0, 2048, (2, 256), device="cuda")
    labels = torch.randint(0, 2048, (2, 256), device="cuda")
    rec = ChunkRecord(len(m.layers))
    logits = model_forward(m, ids, rec)
    loss = torch.nn.functional.cross_entropy(logits.view(-1, 2048).float(), labels.view(-1), reduction="sum")
    model_backward(m, rec, None, loss)
    _native.check_status()
    g1 = {n: p.grad.float().clone() for n, p in m.named_parameters() if p.grad is not None}
    for p in m.parameters():
        p.grad = None
    for mod in m.modules():
        for v in vars(mod).values():
            if type(v).__name__ == "FusedWeights":
                v.fused_grad = None
    fp8_linear.enable(False)  # the oracle is bf16/fp32 math
    logits2 = m.reference_forward(ids)
    loss2 = torch.nn.functional.cross_entropy(logits2.view(-1, 2048).float(), labels.view(-1), reduction="sum")
    loss2.backward()
    assert abs(float(loss) - float(loss2)) / float(loss2) < (2e-2 if fp8 else 5e-3)
    bad = []
    for n, p in m.named_parameters():
        d = calc_diff(g1[n], p.grad.float())
        if d > (8e-2 if fp8 else 2e-2):
            bad.append((n, d))
    assert not bad, bad
