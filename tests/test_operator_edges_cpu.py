"""Edge cases of the operator layer on CPU: activations against eager autograd (saturation, empty inputs), indexed
bias add with empty groups, grouped linear against a per-group loop (empty groups, over-allocated rows, deferred
weight gradients), quantiser corner cases, and a single-process simulation of all expert-parallel ranks.

The same properties are checked by the reference in tests/test_silu_mul.py, tests/test_clamped_swiglu.py,
tests/test_indexed_bias_add.py, tests/test_grouped_linear_correctness.py:330-758,
tests/operators/test_deepgemm_quantize.py:50-381 and tests/test_ep_dedup_dispatch.py:7-253.
"""
import pytest
import torch

from pithtrain_b200.dualpipe.utils import WeightGradStore
from pithtrain_b200.ops import activations as A
from pithtrain_b200.ops import moe as M
from pithtrain_b200.ops import quant as Q
from pithtrain_b200.ops.grouped_linear import GroupedLinear, grouped_linear


def _offsets(sizes):
    return torch.tensor([0] + list(torch.tensor(sizes).cumsum(0)), dtype=torch.int32)


# ------------------------------------------------------------------------------------------------ activations
@pytest.mark.parametrize("dtype,tol", [(torch.float32, 1e-5), (torch.bfloat16, 2e-2)])
def test_silu_mul_matches_eager(dtype, tol):
    torch.manual_seed(0)
    g, u = torch.randn(19, 48).to(dtype).requires_grad_(), torch.randn(19, 48).to(dtype).requires_grad_()
    go = torch.randn(19, 48).to(dtype)
    A.silu_mul(g, u).backward(go)
    got = (g.grad.float(), u.grad.float())
    gf, uf = g.detach().float().requires_grad_(), u.detach().float().requires_grad_()
    ref = torch.nn.functional.silu(gf) * uf
    ref.backward(go.float())
    assert torch.allclose(A.silu_mul(g, u).float(), ref, atol=tol, rtol=tol)
    assert torch.allclose(got[0], gf.grad, atol=tol, rtol=tol) and torch.allclose(got[1], uf.grad, atol=tol, rtol=tol)


def _clamped_swiglu_eager(gu, alpha, limit):
    g, u = gu[..., 0::2], gu[..., 1::2]
    g = g.clamp(max=limit)
    u = u.clamp(min=-limit, max=limit)
    return (u + 1) * g * torch.sigmoid(alpha * g)


def test_clamped_swiglu_matches_eager_and_saturates():
    torch.manual_seed(1)
    gu = (torch.randn(23, 64) * 4).requires_grad_()
    with torch.no_grad():
        gu[0, 0::2] = 9.0  # gate above the limit: clamp(max) has zero slope there
        gu[1, 1::2] = -11.0  # up below -limit
        gu[2, 1::2] = 8.5  # up above +limit
    go = torch.randn(23, 32)
    out = A.clamped_swiglu(gu, 1.702, 7.0)
    out.backward(go)
    ref_in = gu.detach().clone().requires_grad_()
    ref = _clamped_swiglu_eager(ref_in, 1.702, 7.0)
    ref.backward(go)
    assert torch.allclose(out, ref, atol=1e-5, rtol=1e-5)
    assert torch.allclose(gu.grad, ref_in.grad, atol=1e-5, rtol=1e-5)
    assert float(gu.grad[0, 0::2].abs().max()) == 0.0  # saturated gate receives no gradient
    assert float(gu.grad[1, 1::2].abs().max()) == 0.0 and float(gu.grad[2, 1::2].abs().max()) == 0.0


def test_activations_accept_empty_inputs():
    gu = torch.zeros(0, 32, requires_grad=True)
    out = A.clamped_swiglu(gu)
    assert out.shape == (0, 16)
    out.sum().backward()
    assert gu.grad.shape == (0, 32)
    g = torch.zeros(0, 8, requires_grad=True)
    assert A.silu_mul(g, g).shape == (0, 8)


@pytest.mark.parametrize("sizes", [[16, 0, 32, 16], [0, 0, 16], [48]])
def test_indexed_bias_add_with_empty_groups(sizes):
    torch.manual_seed(2)
    offs = _offsets(sizes)
    R, E, H = int(offs[-1]) + 16, len(sizes), 24  # 16 over-allocated rows past the last group
    x = torch.randn(R, H, requires_grad=True)
    bias = torch.nn.Parameter(torch.randn(E, H))
    go = torch.randn(R, H)
    y = A.indexed_bias_add(x, bias, offs)
    y.backward(go)
    got = bias.grad.clone() if bias.grad is not None else bias.main_grad.clone()
    for e in range(E):
        a, b = int(offs[e]), int(offs[e + 1])
        assert torch.allclose(y[a:b], x[a:b] + bias[e])
        assert torch.allclose(got[e], go[a:b].sum(0), atol=1e-5)
    assert torch.equal(x.grad, go)


# ------------------------------------------------------------------------------------------------ grouped linear
def _loop_reference(x, w, offs):
    out = torch.zeros(x.shape[0], w.shape[1])
    for e in range(w.shape[0]):
        a, b = int(offs[e]), int(offs[e + 1])
        out[a:b] = x[a:b] @ w[e].t()
    return out


@pytest.mark.parametrize("sizes,extra", [([16, 32, 0, 16], 0), ([0, 16, 0, 0], 0), ([32, 16, 16, 48], 64), ([0, 0], 32)])
def test_grouped_linear_vs_loop(sizes, extra):
    """Empty groups and rows allocated past the last group (the static capacity bound) leave the result of the
    populated rows and all gradients unchanged."""
    torch.manual_seed(3)
    offs = _offsets(sizes)
    used = int(offs[-1])
    E, K, N = len(sizes), 24, 40
    x = torch.randn(used + extra, K)
    with torch.no_grad():
        x[used:] = 0  # pad rows are zero by construction of the sorted layout
    x.requires_grad_()
    lin = GroupedLinear(E, K, N)
    y = lin(x, offs)
    go = torch.randn(used + extra, N)
    go[used:] = 0
    y.backward(go)
    gw = lin.weight.grad if lin.weight.grad is not None else lin.weight.main_grad
    xr, wr = x.detach().clone().requires_grad_(), lin.weight.detach().clone().requires_grad_()
    ref = _loop_reference(xr, wr, offs)
    ref.backward(go)
    assert torch.allclose(y[:used], ref[:used], atol=1e-5, rtol=1e-5)
    assert torch.allclose(x.grad[:used], xr.grad[:used], atol=1e-5, rtol=1e-5)
    assert torch.allclose(gw, wr.grad, atol=1e-4, rtol=1e-4)


def test_grouped_linear_defers_weight_gradient():
    """With the store enabled the backward returns the input gradient at once and leaves the weight gradient to a
    closure; popping the store produces exactly the eager weight gradient, in FIFO order of the flushes."""
    torch.manual_seed(4)
    offs = _offsets([16, 32])
    w = torch.nn.Parameter(torch.randn(2, 12, 20) * 0.1)
    buf = torch.zeros_like(w)
    xs = [torch.randn(48, 20, requires_grad=True) for _ in range(2)]
    gos = [torch.randn(48, 12) for _ in range(2)]
    WeightGradStore.clear()
    WeightGradStore.enabled = True
    try:
        for x, go in zip(xs, gos):
            grouped_linear(x, w, offs, grad_getter=lambda: buf).backward(go)
            assert x.grad is not None and float(buf.abs().max()) == 0.0
            WeightGradStore.flush()
        WeightGradStore.enabled = False
        WeightGradStore.pop()
        first = buf.clone()
        WeightGradStore.pop()
    finally:
        WeightGradStore.enabled = False
        WeightGradStore.clear()
    wr = w.detach().clone().requires_grad_()
    _loop_reference(xs[0].detach(), wr, offs).backward(gos[0])
    assert torch.allclose(first, wr.grad, atol=1e-5)
    _loop_reference(xs[1].detach(), wr, offs).backward(gos[1])
    assert torch.allclose(buf, wr.grad, atol=1e-5)


# ------------------------------------------------------------------------------------------------ quantisers
def test_quantiser_corner_cases():
    """All-zero input, a width that is not a multiple of 128, and sign symmetry of payload and scales."""
    z = torch.zeros(5, 300).bfloat16()
    q, s = Q.quant_rows_ref(z)
    assert float(q.float().abs().max()) == 0.0 and torch.isfinite(s).all() and bool((s > 0).all())
    assert s.shape == (3, 5)  # ceil(300 / 128) segments, stored segment-major
    qb, sb = Q.quant_blocks_ref(torch.zeros(1, 130, 300).bfloat16())
    assert float(qb.float().abs().max()) == 0.0 and sb.shape == (1, 2, 3) and bool((sb > 0).all())
    torch.manual_seed(5)
    x = (torch.randn(9, 300) * 3).bfloat16()
    qp, sp = Q.quant_rows_ref(x)
    qn, sn = Q.quant_rows_ref(-x)
    assert torch.equal(sp, sn) and torch.equal(qp.float(), -qn.float())
    # the last, partial segment takes its scale from its own 44 columns only
    tail = x[:, 256:].float().abs().amax(1)
    assert torch.equal(sp[2], Q.pow2_scale_ref(tail))
    # scaling the input by a power of two scales the scales, not the payload
    q4, s4 = Q.quant_rows_ref((x.float() * 4).bfloat16())
    assert torch.equal(q4.float(), qp.float()) and torch.equal(s4, sp * 4)


def test_fp8_linear_empty_input_and_deferred_wgrad():
    from pithtrain_b200.ops.linear import linear

    torch.manual_seed(6)
    w = torch.nn.Parameter((torch.randn(256, 256) * 0.05).bfloat16())
    e = torch.zeros(0, 256).bfloat16().requires_grad_()
    y = linear(e, w, fp8=True)
    assert y.shape == (0, 256)
    y.sum().backward()
    assert e.grad.shape == (0, 256)
    g0 = w.grad if w.grad is not None else getattr(w, "main_grad", None)
    assert g0 is None or float(g0.float().abs().max()) == 0.0

    x = torch.randn(32, 256).bfloat16().requires_grad_()
    go = torch.randn(32, 256).bfloat16()
    w.grad = None
    linear(x, w, fp8=True).backward(go)
    eager = (w.grad if w.grad is not None else w.main_grad).float().clone()
    w.grad = None
    if hasattr(w, "main_grad"):
        w.main_grad.zero_()
    WeightGradStore.clear()
    WeightGradStore.enabled = True
    try:
        x2 = x.detach().clone().requires_grad_()
        linear(x2, w, fp8=True).backward(go)
        pending = w.grad if w.grad is not None else getattr(w, "main_grad", None)
        assert pending is None or float(pending.float().abs().max()) == 0.0
        assert torch.equal(x2.grad, x.grad)
        WeightGradStore.flush()
        WeightGradStore.enabled = False
        WeightGradStore.pop()
    finally:
        WeightGradStore.enabled = False
        WeightGradStore.clear()
    deferred = (w.grad if w.grad is not None else w.main_grad).float()
    assert torch.equal(deferred, eager)


# ------------------------------------------------------------------------------------------------ EP simulation
def _simulate_ep_layer(tokens, scores, topk, w1, w2, ep):
    """All ranks of an expert-parallel group in one process: the send side of every rank, the hand-assembled receive
    buffers, the local expert block of every rank, the return trip and the home reduction."""
    from pithtrain_b200.parallel.ep import build_send_side

    E = w1.shape[0]
    epr = E // ep
    sides = [build_send_side(topk[r], E, ep) for r in range(ep)]
    outs = []
    partial_back = [[None] * ep for _ in range(ep)]  # [source][dest]
    for g in range(ep):
        xs, ws, es, owners = [], [], [], []
        for r in range(ep):
            tok, pos, eids, counts = sides[r]
            c = counts.tolist()
            a = sum(c[:g])
            rows = tok[a:a + c[g]].long()
            xs.append(tokens[r][rows]); ws.append(scores[r][rows]); es.append(eids[a:a + c[g]])
            owners.append(c[g])
        x_recv, w_recv, e_recv = torch.cat(xs), torch.cat(ws), torch.cat(es)
        assert e_recv.numel() == 0 or int(e_recv.max()) < epr
        if x_recv.shape[0]:
            part = M.moe_experts_ref(x_recv, w_recv, e_recv, w1[g * epr:(g + 1) * epr], w2[g * epr:(g + 1) * epr])
        else:
            part = x_recv
        at = 0
        for r in range(ep):
            partial_back[r][g] = part[at:at + owners[r]]
            at += owners[r]
    for r in range(ep):
        tok, pos, eids, counts = sides[r]
        back = torch.cat([partial_back[r][g] for g in range(ep)])
        assert back.shape[0] == tok.numel()
        outs.append(M.combine_rows(back.contiguous(), pos.reshape(-1), ep))
    return outs, sides


EP_CASES = [(1, 1, 4, 2), (1, 4, 8, 4), (7, 1, 8, 2), (16, 2, 4, 4), (33, 4, 16, 4), (64, 8, 128, 2),
            (40, 6, 64, 8), (5, 2, 2, 2), (128, 8, 32, 4), (17, 3, 12, 3), (0, 2, 8, 2), (256, 8, 128, 8)]


@pytest.mark.parametrize("m,k,E,ep", EP_CASES)
@pytest.mark.parametrize("seed", [0, 1, 2])
def test_ep_ranks_simulated_in_one_process(m, k, E, ep, seed):
    """De-duplicated dispatch + expert-side weighting + one-row-per-dispatched-row combine reproduce the layer with
    all experts local, for every rank, including m = 0, m = 1 and k = 1."""
    torch.manual_seed(seed)
    H, I = 16, 8
    w1, w2 = torch.randn(E, 2 * I, H) * 0.3, torch.randn(E, H, I) * 0.3
    tokens = [torch.randn(m, H) for _ in range(ep)]
    scores = [torch.rand(m, k) for _ in range(ep)]
    topk = [torch.stack([torch.randperm(E)[:k] for _ in range(m)]).int() if m else torch.zeros(0, k, dtype=torch.int32)
            for _ in range(ep)]
    outs, sides = _simulate_ep_layer(tokens, scores, topk, w1, w2, ep)
    epr = E // ep
    for r in range(ep):
        want = M.moe_experts_ref(tokens[r], scores[r], topk[r], w1, w2) if m else tokens[r]
        assert torch.allclose(outs[r], want, atol=1e-5, rtol=1e-5)
        tok, pos, eids, counts = sides[r]
        dest = topk[r].long() // epr
        # every token travels once per distinct destination rank, never more
        assert tok.numel() == sum(len(set(dest[t].tolist())) for t in range(m))
        assert tok.numel() <= m * min(k, ep)
        # a row carries exactly the local expert ids of its destination, the other slots are masked
        kept = (eids >= 0).sum()
        assert int(kept) == m * k
        if m:
            assert torch.equal(tok[pos[pos >= 0].long()].long(), torch.nonzero(pos >= 0)[:, 0])
