"""tcgen05 GEMM family vs fp32 PyTorch references (dense NT/NN/TN, M-grouped, K-grouped)."""
import os
import pytest
import torch

from pithtrain_b200 import _native
from pithtrain_b200.ops import gemm as G

pytestmark = pytest.mark.gpu


def calc_diff(x, y):
    x, y = x.double(), y.double()
    d = (x * x + y * y).sum()
    return 0.0 if d == 0 else float(1 - 2 * (x * y).sum() / d)


def _rand(*shape):
    return (torch.randn(*shape, device="cuda") * 0.5).to(torch.bfloat16)


@pytest.mark.parametrize("tma_store", [False, True])
@pytest.mark.parametrize("M,N,K", [(128, 128, 64), (256, 256, 128), (384, 512, 192), (1000, 776, 328),
                                   (4096, 2048, 2048), (130, 136, 72)])
def test_dense_nt(M, N, K, tma_store):
    G.USE_TMA_STORE = tma_store
    torch.manual_seed(0)
    x, w = _rand(M, K), _rand(N, K)
    out = G.gemm_nt(x, w)
    _native.check_status()
    ref = x.float() @ w.float().t()
    assert calc_diff(out.float(), ref) < 1e-4
    assert torch.allclose(out.float(), ref, atol=0.25, rtol=2e-2)
    G.USE_TMA_STORE = True


@pytest.mark.parametrize("bn", [128, 256])
def test_dense_bn(bn):
    G.FORCE_BN = bn
    try:
        x, w = _rand(512, 256), _rand(512, 256)
        out = G.gemm_nt(x, w)
        _native.check_status()
        assert calc_diff(out.float(), x.float() @ w.float().t()) < 1e-4
    finally:
        G.FORCE_BN = 0


@pytest.mark.parametrize("M,N,K", [(256, 256, 128), (1000, 776, 328), (4096, 4096, 2048)])
def test_dense_nn(M, N, K):
    dy, w = _rand(M, N), _rand(N, K)
    out = G.gemm_nn(dy, w)
    _native.check_status()
    assert calc_diff(out.float(), dy.float() @ w.float()) < 1e-4


@pytest.fixture(params=[0, 1, 2])
def acc_epilogue(request):
    G.ACC_EPILOGUE = request.param
    yield request.param
    G.ACC_EPILOGUE = 2


@pytest.mark.parametrize("M,N,K", [(256, 256, 128), (1000, 776, 328), (4096, 512, 2048)])
def test_dense_tn(M, N, K, acc_epilogue):
    dy, x = _rand(M, N), _rand(M, K)
    out = G.gemm_tn(dy, x, out_dtype=torch.float32)
    _native.check_status()
    ref = dy.float().t() @ x.float()
    assert calc_diff(out, ref) < 1e-5
    acc = ref.clone()
    G.gemm_tn(dy, x, out=acc, accumulate=True)
    _native.check_status()
    assert calc_diff(acc, 2 * ref) < 1e-5
    accb = ref.to(torch.bfloat16)
    G.gemm_tn(dy, x, out=accb, accumulate=True)
    assert calc_diff(accb.float(), 2 * ref) < 1e-4


def _offsets(sizes):
    o = [0]
    for s in sizes:
        o.append(o[-1] + s)
    return torch.tensor(o, dtype=torch.int32, device="cuda")


@pytest.mark.parametrize("sizes", [[128, 256], [16, 0, 48, 304, 1], [200] * 8, [0, 0, 5], [1024, 16, 640, 0, 272]])
@pytest.mark.parametrize("N,K", [(256, 128), (1536, 2048), (192, 320)])
def test_grouped_nt_nn(sizes, N, K):
    offs = _offsets(sizes)
    R = int(offs[-1]) + 37
    Gn = len(sizes)
    x = _rand(R, K)
    w = _rand(Gn, N, K)
    out = torch.full((R, N), 7.0, dtype=torch.bfloat16, device="cuda")
    G.grouped_gemm_nt(x, w, offs, out=out)
    _native.check_status()
    ref = torch.full((R, N), 7.0, device="cuda")
    for g in range(Gn):
        a, b = int(offs[g]), int(offs[g + 1])
        ref[a:b] = x[a:b].float() @ w[g].float().t()
    assert calc_diff(out.float(), ref) < 1e-4
    assert torch.equal(out[int(offs[-1]):].float(), ref[int(offs[-1]):])
    if N % 64 == 0:
        dy = _rand(R, N)
        dx = torch.full((R, K), 3.0, dtype=torch.bfloat16, device="cuda")
        G.grouped_gemm_nn(dy, w, offs, out=dx)
        _native.check_status()
        ref = torch.full((R, K), 3.0, device="cuda")
        for g in range(Gn):
            a, b = int(offs[g]), int(offs[g + 1])
            ref[a:b] = dy[a:b].float() @ w[g].float()
        assert calc_diff(dx.float(), ref) < 1e-4


@pytest.mark.parametrize("sizes", [[128, 256], [16, 0, 48, 304], [208] * 8, [1024, 16, 640, 0, 272]])
@pytest.mark.parametrize("N,K", [(256, 128), (768, 2048), (192, 320)])
def test_grouped_tn(sizes, N, K, acc_epilogue):
    offs = _offsets(sizes)
    R = int(offs[-1]) + 64
    Gn = len(sizes)
    dy, x = _rand(R, N), _rand(R, K)
    out = torch.randn(Gn, N, K, device="cuda")
    ref = out.clone()
    G.grouped_gemm_tn(dy, x, offs, out, accumulate=True)
    _native.check_status()
    for g in range(Gn):
        a, b = int(offs[g]), int(offs[g + 1])
        ref[g] += dy[a:b].float().t() @ x[a:b].float()
    assert calc_diff(out, ref) < 1e-5
    outb = torch.zeros(Gn, N, K, device="cuda", dtype=torch.bfloat16)
    G.grouped_gemm_tn(dy, x, offs, outb, accumulate=False)
    _native.check_status()
    refb = torch.zeros(Gn, N, K, device="cuda")
    for g in range(Gn):
        a, b = int(offs[g]), int(offs[g + 1])
        refb[g] = dy[a:b].float().t() @ x[a:b].float()
    assert calc_diff(outb.float(), refb) < 1e-4


@pytest.mark.parametrize("sizes1,sizes2", [([128, 256], [64, 16]), ([16, 0, 48, 304], [0, 32, 0, 16]),
                                           ([208] * 8, [1024, 0, 16, 0, 640, 0, 272, 48]), ([0, 0, 64], [0, 0, 0])])
@pytest.mark.parametrize("N,K", [(256, 128), (768, 2048), (192, 320)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_grouped_tn_pair(sizes1, sizes2, N, K, dtype):
    """Two micro-batches' weight gradients in one launch equal the fp32 sum of both products."""
    o1, o2 = _offsets(sizes1), _offsets(sizes2)
    Gn = len(sizes1)
    dy1, x1 = _rand(int(o1[-1]) + 64, N), _rand(int(o1[-1]) + 64, K)
    dy2, x2 = _rand(int(o2[-1]) + 16, N), _rand(int(o2[-1]) + 16, K)
    out = torch.randn(Gn, N, K, device="cuda").to(dtype)
    ref = out.float().clone()
    G.grouped_gemm_tn_pair(dy1, x1, o1, dy2, x2, o2, out)
    _native.check_status()
    for g in range(Gn):
        a, b = int(o1[g]), int(o1[g + 1])
        ref[g] += dy1[a:b].float().t() @ x1[a:b].float()
        a, b = int(o2[g]), int(o2[g + 1])
        ref[g] += dy2[a:b].float().t() @ x2[a:b].float()
    assert calc_diff(out.float(), ref) < (1e-5 if dtype == torch.float32 else 1e-4)


@pytest.mark.parametrize("sizes,N,K", [([256, 0, 128, 400, 16], 512, 256), ([1008, 48, 640], 1536, 2048)])
def test_grouped_gather_matches_explicit_gather(sizes, N, K):
    """The in-kernel TMA row gather equals gather_rows followed by the plain grouped GEMM, bit for bit."""
    offs = _offsets(sizes)
    R = int(offs[-1]) + 48
    n_src, div = 300, 2
    src = _rand(n_src, K)
    idx = torch.randint(0, n_src * div, (R,), device="cuda", dtype=torch.int32)
    idx[::7] = -1
    idx[int(offs[-1]):] = -1
    w = _rand(len(sizes), N, K)
    xs = G._gathered(src, idx, div)
    ref = torch.full((R, N), 5.0, dtype=torch.bfloat16, device="cuda")
    G.grouped_gemm_nt(xs, w, offs, out=ref)
    out = torch.full((R, N), 5.0, dtype=torch.bfloat16, device="cuda")
    G.grouped_gemm_nt(src, w, offs, out=out, a_idx=idx, a_idx_div=div)
    _native.check_status()
    assert torch.equal(out, ref)
    # dgrad form: A gathered, B read MN-major
    srcn = _rand(n_src, N)
    dys = G._gathered(srcn, idx, div)
    ref2 = G.grouped_gemm_nn(dys, w, offs)
    out2 = G.grouped_gemm_nn(srcn, w, offs, a_idx=idx, a_idx_div=div)
    _native.check_status()
    last = int(offs[-1])
    assert torch.equal(out2[:last], ref2[:last])


@pytest.mark.parametrize("M,N,K", [(256, 256, 64), (512, 768, 256), (4096, 5120, 2048), (300, 200, 136)])
def test_two_cta_gemm_nt(M, N, K):
    from pithtrain_b200.ops import gemm as G

    torch.manual_seed(21)
    x = (torch.randn(M, K, device="cuda") * 0.5).bfloat16()
    w = (torch.randn(N, K, device="cuda") * 0.5).bfloat16()
    got = G._gemm2cta_nt(x, w).float()
    torch.cuda.synchronize()
    _native.check_status()
    ref = x.float() @ w.float().t()
    assert calc_diff(got, ref) < 1e-4
