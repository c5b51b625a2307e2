"""The own tcgen05 attention kernels against the fp32 math (``attention_ref``): forward output and log-sum-exp,
backward dq / dk / dv (and sink gradients), over the masks and head dims the model families use."""

import pytest
import torch

from pithtrain_b200 import _native
from pithtrain_b200.ops import attention as A
from pithtrain_b200.ops import attention_native as N
from utilities import calc_diff

pytestmark = pytest.mark.gpu


def _qkv(B, Sq, Sk, Hq, Hkv, D, Dv, seed=0, fused=True):
    torch.manual_seed(seed)
    if fused and Sq == Sk:
        # slices of one projection output, like the model's fused qkv projection
        qkv = torch.randn(B, Sq, Hq * D + Hkv * D + Hkv * Dv, device="cuda").bfloat16()
        q = qkv[..., :Hq * D].view(B, Sq, Hq, D)
        k = qkv[..., Hq * D:(Hq + Hkv) * D].view(B, Sq, Hkv, D)
        v = qkv[..., (Hq + Hkv) * D:].view(B, Sq, Hkv, Dv)
    else:
        q = torch.randn(B, Sq, Hq, D, device="cuda").bfloat16()
        k = torch.randn(B, Sk, Hkv, D, device="cuda").bfloat16()
        v = torch.randn(B, Sk, Hkv, Dv, device="cuda").bfloat16()
    return q, k, v


def _check_fwd(q, k, v, causal=True, window=None, sinks=None, cu=None, tol=2e-4):
    assert N.supported(q, k, v, causal, window, sinks, cu)
    out, lse = N.attention(q, k, v, causal, None, window, sinks, cu, return_lse=True)
    torch.cuda.synchronize()
    _native.check_status()
    ref, ref_lse = A.attention_ref(q, k, v, causal, None, window, sinks, cu, return_lse=True)
    assert calc_diff(out.float(), ref.float()) < tol
    fin = torch.isfinite(ref_lse)
    assert torch.allclose(lse[fin], ref_lse[fin], atol=2e-2, rtol=1e-3)


@pytest.mark.parametrize("B,S,Hq,Hkv,D,Dv", [
    (1, 256, 4, 2, 128, 128), (2, 1024, 8, 2, 128, 128), (1, 4096, 8, 1, 128, 128), (1, 384, 4, 4, 128, 128),
    (2, 512, 8, 2, 64, 64), (1, 512, 4, 4, 192, 128), (1, 512, 4, 2, 256, 256), (2, 200, 4, 2, 128, 128),
])
def test_causal_forward(B, S, Hq, Hkv, D, Dv):
    q, k, v = _qkv(B, S, S, Hq, Hkv, D, Dv, seed=1)
    _check_fwd(q, k, v)


@pytest.mark.parametrize("Sq,Sk,causal", [(256, 384, False), (256, 512, True), (128, 1024, False), (300, 300, False)])
def test_block_forward_sq_ne_sk(Sq, Sk, causal):
    q, k, v = _qkv(1, Sq, Sk, 8, 2, 128, 128, seed=2, fused=False)
    _check_fwd(q, k, v, causal=causal)


@pytest.mark.parametrize("D", [64, 128])
def test_window_sinks_and_documents_forward(D):
    S, Hq, Hkv = 1024, 8, 2
    q, k, v = _qkv(1, S, S, Hq, Hkv, D, D, seed=3)
    sinks = torch.randn(Hq, device="cuda").bfloat16()
    _check_fwd(q, k, v, window=127, sinks=sinks)
    _check_fwd(q, k, v, sinks=sinks)
    cu = torch.tensor([0, 100, 300, 777, S], dtype=torch.int32, device="cuda")
    _check_fwd(q, k, v, cu=cu)
    _check_fwd(q, k, v, window=200, cu=cu, sinks=sinks)


def _check_bwd(q, k, v, causal=True, window=None, sinks=None, cu=None, tol=5e-4):
    q, k, v = (t.detach().clone().requires_grad_() for t in (q, k, v))
    sk = None if sinks is None else sinks.detach().clone().requires_grad_()
    out = N.attention(q, k, v, causal, None, window, sk, cu)
    go = torch.randn_like(out)
    ins = [q, k, v] + ([sk] if sk is not None else [])
    got = torch.autograd.grad(out, ins, go)
    torch.cuda.synchronize()
    _native.check_status()
    q2, k2, v2 = (t.detach().clone().requires_grad_() for t in (q, k, v))
    sk2 = None if sinks is None else sinks.detach().clone().requires_grad_()
    ref = A.attention_ref(q2, k2, v2, causal, None, window, sk2, cu)
    want = torch.autograd.grad(ref, [q2, k2, v2] + ([sk2] if sk2 is not None else []), go)
    for name, a, b in zip(("dq", "dk", "dv", "dsinks"), got, want):
        assert calc_diff(a.float(), b.float()) < tol, name


@pytest.mark.parametrize("B,S,Hq,Hkv,D", [
    (1, 128, 1, 1, 128), (1, 256, 2, 1, 128), (2, 1024, 8, 2, 128), (1, 2048, 8, 1, 128), (2, 512, 8, 2, 64),
    (2, 200, 4, 2, 128),
])
def test_causal_backward(B, S, Hq, Hkv, D):
    q, k, v = _qkv(B, S, S, Hq, Hkv, D, D, seed=4)
    _check_bwd(q, k, v)


@pytest.mark.parametrize("Sq,Sk,causal", [(256, 384, False), (256, 512, True), (300, 300, False)])
def test_block_backward_sq_ne_sk(Sq, Sk, causal):
    q, k, v = _qkv(1, Sq, Sk, 8, 2, 128, 128, seed=5, fused=False)
    _check_bwd(q, k, v, causal=causal)


@pytest.mark.parametrize("D", [64, 128])
def test_window_sinks_and_documents_backward(D):
    S, Hq, Hkv = 1024, 8, 2
    q, k, v = _qkv(1, S, S, Hq, Hkv, D, D, seed=6)
    sinks = torch.randn(Hq, device="cuda").bfloat16()
    _check_bwd(q, k, v, window=127, sinks=sinks)
    _check_bwd(q, k, v, sinks=sinks)
    cu = torch.tensor([0, 100, 300, 777, S], dtype=torch.int32, device="cuda")
    _check_bwd(q, k, v, cu=cu)
    _check_bwd(q, k, v, window=200, cu=cu, sinks=sinks)


def test_mla_and_wide_heads_differentiate_through_math():
    q, k, v = _qkv(1, 256, 256, 4, 4, 192, 128, seed=7)
    _check_bwd(q, k, v)
    q, k, v = _qkv(1, 256, 256, 4, 2, 256, 256, seed=8)
    _check_bwd(q, k, v)
