"""FP8 kernels on a B200: quantisers bit-exact against the tensor-op restatement, block-scaled GEMM against
an fp32 matmul of the de-quantised operands, and the fp8 expert block against the bf16 one."""
import pytest
import torch

from pithtrain_b200.ops import fp8_linear as F8
from pithtrain_b200.ops import quant as Q
from utilities import calc_diff

pytestmark = pytest.mark.gpu
DEV = "cuda"


@pytest.mark.parametrize("R,K", [(300, 2048), (129, 2880), (4096, 768), (17, 136)])
def test_quant_rows_bit_exact(R, K):
    from pithtrain_b200 import _native

    torch.manual_seed(R + K)
    x = (torch.randn(R, K, device=DEV) * torch.logspace(-4, 3, R, device=DEV).unsqueeze(1)).bfloat16()
    x[R // 2] = 0
    q, s = Q.quant_rows(x)
    qr, sr = Q.quant_rows_ref(x)
    _native.check_status()
    assert torch.equal(s[:, :R], sr)
    assert torch.equal(q.view(torch.uint8), qr.view(torch.uint8))
    idx = torch.randint(-1, 2 * R, (R + 40,), device=DEV, dtype=torch.int32)
    n_rows = torch.tensor([R + 8], device=DEV, dtype=torch.int32)
    qg, sg = Q.quant_rows(x, idx=idx, div=2, n_rows=n_rows)
    src = torch.where((idx >= 0).unsqueeze(1), x[(idx.clamp(min=0) // 2).long()], torch.zeros((), device=DEV, dtype=x.dtype))
    qr, sr = Q.quant_rows_ref(src[:R + 8])
    assert torch.equal(qg[:R + 8].view(torch.uint8), qr.view(torch.uint8)) and torch.equal(sg[:, :R + 8], sr)


@pytest.mark.parametrize("G,N,K", [(1, 512, 2048), (3, 200, 300), (4, 1536, 2048), (2, 2880, 2880)])
def test_quant_blocks_bit_exact(G, N, K):
    torch.manual_seed(G * N + K)
    w = (torch.randn(G, N, K, device=DEV) * 0.05).bfloat16()
    q, s, qt, st = Q.quant_blocks(w)
    qr, sr = Q.quant_blocks_ref(w)
    assert torch.equal(s, sr) and torch.equal(st, sr.transpose(1, 2))
    assert torch.equal(q.view(torch.uint8), qr.view(torch.uint8))
    assert torch.equal(qt.view(torch.uint8), qr.transpose(1, 2).contiguous().view(torch.uint8))


@pytest.mark.parametrize("M,N,K", [(256, 256, 256), (4096, 5120, 2048), (1000, 2880, 2880), (333, 776, 1408), (128, 128, 128)])
@pytest.mark.parametrize("tma", [True, False])
def test_gemm_fp8_dense(M, N, K, tma):
    from pithtrain_b200 import _native

    torch.manual_seed(M + N + K)
    x = torch.randn(M, K, device=DEV).bfloat16()
    w = (torch.randn(N, K, device=DEV) * 0.05).bfloat16()
    xq, xs = Q.quant_rows(x)
    wq, ws, _, _ = Q.quant_blocks(w, transposed=False)
    y = Q.gemm_fp8_nt(xq, xs, wq, ws, use_tma_store=tma)
    _native.check_status()
    ref = Q.dequant_rows(xq, xs) @ Q.dequant_blocks(wq, ws)[0].t()
    assert calc_diff(y.float(), ref) < 1e-5
    assert torch.allclose(y.float(), ref, atol=2e-2 * float(ref.abs().max()), rtol=2e-2)
    assert calc_diff(y.float(), x.float() @ w.float().t()) < 2e-3  # fp8 against the unquantised product


@pytest.mark.parametrize("E,H,N", [(8, 2048, 1536), (5, 768, 2048), (4, 2880, 5760)])
def test_gemm_fp8_grouped(E, H, N):
    from pithtrain_b200 import _native

    torch.manual_seed(E + H)
    sizes = torch.tensor([0, 16, 400, 128, 1008, 48, 256, 640][:E]) if E <= 8 else None
    offs = torch.cat([torch.zeros(1, dtype=torch.long), sizes.cumsum(0)]).int().to(DEV)
    R = int(offs[-1]) + 64  # capacity past the last group stays untouched
    x = torch.randn(R, H, device=DEV).bfloat16()
    w = (torch.randn(E, N, H, device=DEV) * 0.05).bfloat16()
    xq, xs = Q.quant_rows(x, n_rows=offs[E:E + 1])
    wq, ws, wqt, wst = Q.quant_blocks(w)
    y = torch.full((R, N), 7.0, device=DEV, dtype=torch.bfloat16)
    Q.gemm_fp8_nt(xq, xs, wq, ws, offs=offs, out=y)
    _native.check_status()
    a, b = Q.dequant_rows(xq, xs), Q.dequant_blocks(wq, ws)
    o = offs.tolist()
    for g in range(E):
        if o[g + 1] > o[g]:
            ref = a[o[g]:o[g + 1]] @ b[g].t()
            assert calc_diff(y[o[g]:o[g + 1]].float(), ref) < 1e-5, g
    assert bool((y[o[E]:] == 7.0).all())
    # transposed weights give the input-gradient product
    dy = torch.randn(R, N, device=DEV).bfloat16()
    dq, ds = Q.quant_rows(dy, n_rows=offs[E:E + 1])
    dx = Q.gemm_fp8_nt(dq, ds, wqt, wst, offs=offs)
    g = 2
    ref = dy[o[g]:o[g + 1]].float() @ w[g].float()
    assert calc_diff(dx[o[g]:o[g + 1]].float(), ref) < 2e-3


def test_fp8_expert_block_matches_bf16_block():
    from pithtrain_b200.ops import moe as M

    torch.manual_seed(5)
    n, k, E, H, I = 1024, 4, 8, 2048, 768
    eids = torch.stack([torch.randperm(E)[:k] for _ in range(n)]).int().to(DEV)
    w1, w2 = (torch.randn(E, 2 * I, H, device=DEV) * 0.03).bfloat16(), (torch.randn(E, H, I, device=DEV) * 0.03).bfloat16()
    outs = []
    for flag in (False, True):
        F8.enable(flag)
        try:
            x = torch.randn(n, H, device=DEV, generator=torch.Generator(DEV).manual_seed(3)).bfloat16().requires_grad_()
            w = torch.rand(n, k, device=DEV, generator=torch.Generator(DEV).manual_seed(4)).requires_grad_()
            g1, g2 = torch.zeros_like(w1), torch.zeros_like(w2)
            out = M.moe_experts(x, w, eids, M.ExpertWeights(w1, w2, lambda: g1, lambda: g2))
            out.float().square().mean().backward()
            outs.append((out.detach().float(), x.grad.float(), w.grad.float(), g1.float(), g2.float()))
        finally:
            F8.enable(False)
    for a, b in zip(*outs):
        assert calc_diff(a, b) < 5e-3


def test_fp8_linear_module():
    from pithtrain_b200.ops.linear import Linear

    torch.manual_seed(6)
    lin = F8.FP8Linear(2048, 4096, bias=True, device=DEV, dtype=torch.bfloat16)
    ref = Linear(2048, 4096, bias=True, device=DEV, dtype=torch.bfloat16)
    ref.load_state_dict(lin.state_dict())
    x = torch.randn(2, 512, 2048, device=DEV).bfloat16()
    outs = []
    for m in (lin, ref):
        xi = x.clone().requires_grad_()
        y = m(xi)
        y.float().square().mean().backward()
        g = m.weight.grad if m.weight.grad is not None else m.weight.main_grad
        outs.append((y.detach().float(), xi.grad.float(), g.float()))
    for a, b in zip(*outs):
        assert calc_diff(a, b) < 3e-3
