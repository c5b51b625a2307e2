"""FP8 recipe on CPU: scale rule, quantiser round trips, fp8 linear / expert block against bf16 math."""
import torch

from pithtrain_b200.ops import fp8_linear as F8
from pithtrain_b200.ops import quant as Q


def test_pow2_scale_rule():
    amax = torch.tensor([0.0, 1e-5, 448.0, 448.0001, 1.0, 7.0 * 64, 3e38, 2.0 ** -20 * 448])
    s = Q.pow2_scale_ref(amax)
    # exact powers of two of amax/448 stay; everything else rounds up; floor at 1e-4/448
    assert s[2] == 1.0 and s[3] == 2.0 and s[5] == 1.0 and s[7] == 2.0 ** -20
    floor = Q.pow2_scale_ref(torch.tensor([1e-4]))
    assert s[0] == floor and s[1] == floor
    assert torch.all(torch.log2(s) == torch.log2(s).round())
    assert torch.all(amax[2:7] / s[2:7] <= 448.0)


def test_quantisers_round_trip():
    torch.manual_seed(0)
    x = (torch.randn(37, 320) * torch.logspace(-3, 2, 37).unsqueeze(1)).bfloat16()
    q, s = Q.quant_rows_ref(x)
    assert q.shape == (37, 320) and s.shape == (3, 37)
    back = Q.dequant_rows(q, s)
    err = (back - x.float()).abs() / x.float().abs().clamp(min=1e-6)
    big = x.float().abs() > (s.t().repeat_interleave(128, 1)[:, :320] * 2 ** -6)  # e4m3 normal range
    assert float(err[big].max()) <= 2 ** -4 + 1e-6  # 3 mantissa bits
    w = torch.randn(2, 200, 300).bfloat16()
    qw, sw = Q.quant_blocks_ref(w)
    assert qw.shape == w.shape and sw.shape == (2, 2, 3)
    assert float((Q.dequant_blocks(qw, sw) - w.float()).abs().max()) < 0.3
    q2, s2, qt, st = Q.quant_blocks(w)
    assert torch.equal(q2.float(), qw.float()) and torch.equal(qt.float(), qw.transpose(1, 2).float())
    assert torch.equal(st, sw.transpose(1, 2))
    # gather + divide index convention
    idx = torch.tensor([6, -1, 0, 5], dtype=torch.int32)
    qg, sg = Q.quant_rows(x, idx=idx, div=2)
    ref, _ = Q.quant_rows_ref(x[[3, 0, 0, 2]])
    assert torch.equal(qg[[0, 2, 3]].float(), ref[[0, 2, 3]].float()) and float(qg[1].float().abs().max()) == 0


def test_fp8_linear_matches_bf16_closely():
    torch.manual_seed(1)
    x = torch.randn(64, 256).bfloat16().requires_grad_()
    w = torch.nn.Parameter((torch.randn(384, 256) * 0.05).bfloat16())
    from pithtrain_b200.ops.linear import linear

    y = linear(x, w, fp8=True)
    y.float().square().mean().backward()
    gx, gw = x.grad.clone(), w.grad.clone() if w.grad is not None else w.main_grad.clone()
    x.grad = None
    ref = torch.nn.functional.linear(x.float(), w.float())
    from tests.utilities import calc_diff

    assert calc_diff(y.float(), ref) < 2e-3
    ref.square().mean().backward()
    assert calc_diff(gx.float(), x.grad.float()) < 5e-3
    assert not F8.enabled() and not F8.eligible(x, w) and F8.eligible(x, w, True)
    assert not F8.eligible(x, torch.zeros(128, 256).bfloat16(), True)  # narrow projections stay bf16


def test_fp8_expert_block_close_to_bf16():
    from pithtrain_b200.ops import moe as M
    from tests.utilities import calc_diff

    torch.manual_seed(2)
    n, k, E, H, I = 96, 2, 4, 256, 256
    eids = torch.stack([torch.randperm(E)[:k] for _ in range(n)]).int()
    w1, w2 = (torch.randn(E, 2 * I, H) * 0.05).bfloat16(), (torch.randn(E, H, I) * 0.05).bfloat16()
    outs = []
    for flag in (False, True):
        F8.enable(flag)
        try:
            x, w = torch.randn(n, H, generator=torch.Generator().manual_seed(3)).bfloat16().requires_grad_(), \
                torch.rand(n, k, generator=torch.Generator().manual_seed(4)).requires_grad_()
            g1, g2 = torch.zeros_like(w1), torch.zeros_like(w2)
            ew = M.ExpertWeights(w1, w2, lambda: g1, lambda: g2)
            out = M.moe_experts(x, w, eids, ew)
            out.float().square().mean().backward()
            outs.append((out.detach().float(), x.grad.float(), w.grad.float(), g1.float(), g2.float()))
        finally:
            F8.enable(False)
    for a, b in zip(*outs):
        assert calc_diff(a, b) < 1e-2


def test_fp8_gradients_feed_muon():
    """fp8 forward/backward produces finite gradients that the Muon update accepts (smoke test of the combination)."""
    from pithtrain_b200.modules.optimizer import Muon
    from pithtrain_b200.ops.linear import Linear

    torch.manual_seed(5)
    lin = F8.FP8Linear(256, 256, bias=False, dtype=torch.bfloat16)
    ref = Linear(256, 256, bias=False, dtype=torch.bfloat16)
    ref.load_state_dict(lin.state_dict())
    opt = Muon([lin.weight], lr=0.05, momentum=0.9, weight_decay=0.0)
    before = lin.weight.detach().clone()
    for _ in range(2):
        y = lin(torch.randn(32, 256).bfloat16())
        y.float().square().mean().backward()
        assert torch.isfinite(lin.weight.grad.float()).all()
        opt.step()
        opt.zero_grad()
        from pithtrain_b200.dualpipe.utils import FP8WeightCacheControl

        FP8WeightCacheControl.step()  # weights changed: cached quantised copies are stale
    assert torch.isfinite(lin.weight.float()).all() and not torch.equal(before, lin.weight.detach())


def test_reference_named_quantiser_wrappers():
    """Output shapes and contents of the casts under the reference's names (pithtrain/operators/deepgemm_quantize.py)."""
    from pithtrain_b200.ops import deepgemm_quantize as DQ

    torch.manual_seed(7)
    x = (torch.randn(256, 300) * 2).bfloat16()
    tok, tok_s, ch, ch_s = DQ.fp8cast_rowwise_colwise(x)
    assert tok.shape == (256, 300) and tok_s.shape == (256, 3) and ch.shape == (256, 300) and ch_s.shape == (2, 300)
    q_ref, s_ref = Q.quant_rows_ref(x)
    assert torch.equal(tok.float(), q_ref.float()) and torch.equal(tok_s, s_ref.t())
    # column-wise: every 128x1 column segment has its own power-of-two scale
    seg = x.float().view(2, 128, 300).abs().amax(1)
    assert torch.equal(ch_s, Q.pow2_scale_ref(seg))
    assert torch.equal(ch.float(), (x.float().view(2, 128, 300) / ch_s[:, None, :]).view(256, 300).to(torch.float8_e4m3fn).float())
    _, _, t, t_s = DQ.fp8cast_rowwise_transpose(x)
    assert t.shape == (300, 256) and t_s.shape == (300, 2) and torch.equal(t.float(), ch.t().float())
    _, _, bt, bt_s = DQ.fp8cast_rowwise_blockwise_transpose(x)
    assert bt.shape == (300, 256) and bt_s.shape == (3, 2)
    q, s, qt, st = DQ.fp8cast_blockwise_transpose(x)
    assert q.shape == (256, 300) and s.shape == (2, 3) and qt.shape == (300, 256) and st.shape == (3, 2)
    assert torch.equal(qt.float(), bt.float()) and torch.equal(st, bt_s) and torch.equal(qt.float(), q.t().float())
    q3, s3, q3t, s3t = DQ.fp8cast_blockwise_transpose_batched(torch.stack([x, -x]))
    assert q3.shape == (2, 256, 300) and s3t.shape == (2, 3, 2) and torch.equal(q3[0].float(), -q3[1].float())
    offs = torch.tensor([128, 256], dtype=torch.int32)
    _, _, flat, km_s = DQ.fp8cast_rowwise_kmajor(x, offs)
    assert flat.shape == (256 * 300,) and km_s.shape == (300, 2)
    assert torch.equal(flat[:128 * 300].view(300, 128).float(), ch[:128].t().float())
    assert torch.equal(flat[128 * 300:].view(300, 128).float(), ch[128:].t().float())
    # uneven groups, an empty one, and rows past the last offset (a trailing block)
    _, _, flat2, _ = DQ.fp8cast_rowwise_kmajor(x, torch.tensor([128, 128, 128 + 64], dtype=torch.int32))
    assert torch.equal(flat2[:128 * 300].view(300, 128).float(), ch[:128].t().float())
    assert torch.equal(flat2[128 * 300:192 * 300].view(300, 64).float(), ch[128:192].t().float())
    assert torch.equal(flat2[192 * 300:].view(300, 64).float(), ch[192:].t().float())
