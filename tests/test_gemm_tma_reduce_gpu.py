"""Weight-gradient epilogue that lets the copy engine accumulate (TMA reduce-add) vs fp32 references."""
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


@pytest.fixture(autouse=True)
def tma_reduce_mode():
    G.ACC_EPILOGUE = 2
    yield
    G.ACC_EPILOGUE = 2


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("M,N,K", [(256, 256, 128), (1000, 776, 328), (4096, 512, 2048)])
def test_dense_tn_tma_reduce(M, N, K, dtype):
    dy, x = _rand(M, N), _rand(M, K)
    ref = dy.float().t() @ x.float()
    acc = ref.to(dtype).clone()
    G.gemm_tn(dy, x, out=acc, accumulate=True)
    _native.check_status()
    assert calc_diff(acc.float(), 2 * ref) < (1e-5 if dtype == torch.float32 else 1e-4)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("sizes", [[128, 256], [16, 0, 48, 304], [208] * 8])
@pytest.mark.parametrize("N,K", [(256, 128), (768, 2048), (192, 320)])
def test_grouped_tn_tma_reduce(sizes, N, K, dtype):
    o = [0]
    for s in sizes:
        o.append(o[-1] + s)
    offs = torch.tensor(o, dtype=torch.int32, device="cuda")
    R, Gn = o[-1] + 64, len(sizes)
    dy, x = _rand(R, N), _rand(R, K)
    out = torch.randn(Gn, N, K, device="cuda").to(dtype)
    ref = out.float().clone()
    G.grouped_gemm_tn(dy, x, offs, out, accumulate=True)
    _native.check_status()
    for g in range(Gn):
        ref[g] += dy[o[g]:o[g + 1]].float().t() @ x[o[g]:o[g + 1]].float()
    assert calc_diff(out.float(), ref) < (1e-5 if dtype == torch.float32 else 1e-4)
