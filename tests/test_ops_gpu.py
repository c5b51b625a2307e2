"""Memory-bound sm_100a kernels vs fp32 PyTorch references."""
import os
import pytest
import torch

from pithtrain_b200 import _native
from pithtrain_b200.ops import moe as M
from pithtrain_b200.ops.cross_entropy import cross_entropy
from pithtrain_b200.ops.norm import rmsnorm, rmsnorm_ref
from pithtrain_b200.ops.rope import qk_norm_rope, qk_norm_rope_ref
from pithtrain_b200.ops.router import router_topk, router_topk_ref

pytestmark = pytest.mark.gpu


def calc_diff(x, y):
    x, y = x.double(), y.double()
    d = (x * x + y * y).sum()
    return 0.0 if d == 0 else float(1 - 2 * (x * y).sum() / d)


def bf(*shape, scale=1.0):
    return (torch.randn(*shape, device="cuda") * scale).to(torch.bfloat16)


@pytest.mark.parametrize("n,H", [(33, 2048), (4096, 2048), (7, 2880), (128, 512), (65, 7168)])
@pytest.mark.parametrize("residual", [False, True])
def test_rmsnorm(n, H, residual):
    torch.manual_seed(0)
    x = bf(n, H).requires_grad_()
    r = bf(n, H).requires_grad_() if residual else None
    w = (1 + 0.1 * torch.randn(H, device="cuda")).to(torch.bfloat16).requires_grad_()
    out = rmsnorm(x, w, 1e-6, r)
    xr, rr, wr = x.detach().float().requires_grad_(), (r.detach().float().requires_grad_() if residual else None), w.detach().float().requires_grad_()
    ref = rmsnorm_ref(xr, wr, 1e-6, rr)
    if residual:
        y, h = out
        yr, hr = ref
        gy, gh = bf(n, H), bf(n, H)
        torch.autograd.backward([y, h], [gy, gh])
        torch.autograd.backward([yr, hr], [gy.float(), gh.float()])
        assert calc_diff(h.float(), hr) < 1e-5
        assert calc_diff(r.grad.float(), rr.grad) < 1e-4
    else:
        y, yr = out, ref
        gy = bf(n, H)
        y.backward(gy)
        yr.backward(gy.float())
    _native.check_status()
    assert calc_diff(y.float(), yr) < 1e-4
    assert calc_diff(x.grad.float(), xr.grad) < 1e-4
    assert calc_diff(w.grad.float(), wr.grad) < 1e-3


@pytest.mark.parametrize("D,Hq,Hkv", [(128, 32, 4), (64, 8, 8), (128, 4, 1)])
@pytest.mark.parametrize("norm", [True, False])
def test_qk_norm_rope(D, Hq, Hkv, norm):
    torch.manual_seed(1)
    B, S = 2, 96
    n = B * S
    qkv = bf(n, (Hq + 2 * Hkv) * D).requires_grad_()
    qw = (1 + 0.1 * torch.randn(D, device="cuda")).to(torch.bfloat16).requires_grad_() if norm else None
    kw = (1 + 0.1 * torch.randn(D, device="cuda")).to(torch.bfloat16).requires_grad_() if norm else None
    t = torch.arange(256, device="cuda", dtype=torch.float32)
    inv = 1.0 / (1e6 ** (torch.arange(0, D, 2, device="cuda", dtype=torch.float32) / D))
    fr = torch.outer(t, inv)
    emb = torch.cat([fr, fr], -1)
    cos, sin = emb.cos().to(torch.bfloat16), emb.sin().to(torch.bfloat16)
    pos = torch.randint(0, 256, (n,), device="cuda", dtype=torch.int32)
    q, k, v = qk_norm_rope(qkv, qw, kw, cos, sin, Hq, Hkv, D, 1e-6, positions=pos, S=S)
    qkv_r = qkv.detach().float().requires_grad_()
    qw_r = qw.detach().float().requires_grad_() if norm else None
    kw_r = kw.detach().float().requires_grad_() if norm else None
    qr, kr, vr = qk_norm_rope_ref(qkv_r, qw_r, kw_r, cos.float(), sin.float(), Hq, Hkv, D, 1e-6, pos, S)
    gq, gk, gv = bf(n, Hq, D), bf(n, Hkv, D), bf(n, Hkv, D)
    torch.autograd.backward([q, k, v], [gq, gk, gv])
    torch.autograd.backward([qr, kr, vr], [gq.float(), gk.float(), gv.float()])
    _native.check_status()
    assert calc_diff(q.float(), qr) < 1e-4 and calc_diff(k.float(), kr) < 1e-4
    assert torch.equal(v.float(), vr)
    assert calc_diff(qkv.grad.float(), qkv_r.grad) < 1e-4
    if norm:
        assert calc_diff(qw.grad.float(), qw_r.grad) < 1e-3
        assert calc_diff(kw.grad.float(), kw_r.grad) < 1e-3


@pytest.mark.parametrize("n,E,k", [(1000, 128, 8), (64, 64, 6), (33, 32, 4), (5, 256, 8)])
@pytest.mark.parametrize("mode,renorm", [("softmax_topk", True), ("softmax_topk", False), ("topk_softmax", False)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_router(n, E, k, mode, renorm, dtype):
    torch.manual_seed(2)
    logits = torch.randn(n, E, device="cuda").to(dtype).requires_grad_()
    w, idx, probs = router_topk(logits, k, mode, renorm, 1.5)
    lr = logits.detach().float().requires_grad_()
    wr, idxr, probsr = router_topk_ref(lr, k, mode, renorm, 1.5)
    # same expert sets; compare weights after aligning by expert id
    si, sir = idx.long().sort(-1), idxr.long().sort(-1)
    same = (si.values == sir.values).all(-1)
    assert same.float().mean() > 0.98  # bf16 ties may differ
    wa, wra = w.gather(-1, si.indices), wr.gather(-1, sir.indices)
    assert torch.allclose(wa[same], wra[same], atol=2e-3, rtol=2e-2)
    gw = torch.randn(n, k, device="cuda")
    gp = torch.randn(n, E, device="cuda") * 0.1 if probs is not None else None
    # gradient check on rows where selections agree, with the upstream grads aligned by expert
    gwa = torch.zeros_like(gw).scatter_(-1, si.indices, gw.gather(-1, si.indices))
    outs, gs = [w], [gwa]
    outs_r, gs_r = [wr], [torch.zeros_like(gw).scatter_(-1, sir.indices, gw.gather(-1, si.indices))]
    if probs is not None:
        outs.append(probs); gs.append(gp); outs_r.append(probsr); gs_r.append(gp)
    torch.autograd.backward(outs, gs)
    torch.autograd.backward(outs_r, gs_r)
    _native.check_status()
    assert calc_diff(logits.grad.float()[same], lr.grad[same]) < (1e-3 if dtype == torch.float32 else 2e-2)


@pytest.mark.parametrize("n,k,E", [(512, 8, 128), (100, 2, 8), (1, 1, 4), (4096, 8, 32), (37, 4, 16)])
def test_route_sort_and_gather_combine(n, k, E):
    torch.manual_seed(3)
    eids = torch.randint(-1, E, (n, k), device="cuda", dtype=torch.int32)
    offs, ros, sor = M.route_sort(eids, E)
    offs_r, ros_r, sor_r = M.route_sort_ref(eids.cpu(), E, sor.numel())
    _native.check_status()
    assert torch.equal(offs.cpu(), offs_r)
    assert torch.equal(ros.cpu(), ros_r)
    end = int(offs[-1])
    assert torch.equal(sor.cpu()[:end], sor_r[:end]) and bool((sor[end:] == -1).all())
    H = 256
    x = bf(n, H)
    xs = M.gather_rows(x, sor, div=k, n_rows=offs[E:E + 1])
    ref = x[(sor[:end].clamp(min=0) // k).long()] * (sor[:end] >= 0).unsqueeze(-1)
    assert torch.equal(xs[:end], ref)
    y = bf(sor.numel(), H)
    w = torch.rand(n, k, device="cuda")
    res = bf(n, H)
    out = M.combine_rows(y, ros, k, w=w, residual=res)
    r = ros.view(n, k).long()
    ref = (y[r.clamp(min=0)].float() * (r >= 0).unsqueeze(-1) * w.unsqueeze(-1)).sum(1) + res.float()
    _native.check_status()
    assert calc_diff(out.float(), ref) < 1e-5


@pytest.mark.parametrize("interleaved,limit", [(False, 0.0), (True, 7.0)])
def test_swiglu(interleaved, limit):
    torch.manual_seed(4)
    R, I = 300, 768
    gu = bf(R, 2 * I, scale=3.0)
    alpha = 1.702 if limit > 0 else 1.0
    act = M.swiglu_fwd(gu, None, interleaved, alpha, limit)
    g, u = M._split_gu(gu.float(), interleaved)
    ref = M._swiglu_math(g, u, alpha, limit)
    assert calc_diff(act.float(), ref) < 1e-5
    dact = bf(R, I)
    rw = torch.rand(R, device="cuda")
    dgu, act_s, dw = M.swiglu_bwd(gu, dact, rw, None, interleaved, alpha, limit, want_act=True, want_dw=True)
    dgu_r, act_r, dw_r = M.swiglu_bwd(gu.cpu(), dact.cpu(), rw.cpu(), None, interleaved, alpha, limit, want_act=True, want_dw=True)
    _native.check_status()
    assert calc_diff(dgu.float().cpu(), dgu_r.float()) < 1e-4
    assert calc_diff(act_s.float().cpu(), act_r.float()) < 1e-4
    assert calc_diff(dw.cpu(), dw_r) < 1e-4


@pytest.mark.parametrize("n,V", [(64, 4096), (37, 151936), (8, 1000)])
def test_cross_entropy(n, V):
    torch.manual_seed(5)
    Vp = (V + 7) // 8 * 8
    buf = bf(n, Vp, scale=2.0)
    logits = buf[:, :V].detach().requires_grad_()
    labels = torch.randint(0, V, (n,), device="cuda")
    labels[::5] = -100
    ref_in = logits.detach().float().requires_grad_()
    ref = torch.nn.functional.cross_entropy(ref_in, labels, ignore_index=-100, reduction="sum")
    (ref * 0.5).backward()
    x = logits.clone().requires_grad_() if False else logits
    loss = cross_entropy(x * 1.0, labels)
    (loss * 0.5).backward()
    _native.check_status()
    assert abs(float(loss) - float(ref)) / abs(float(ref)) < 2e-3
    assert calc_diff(logits.grad.float(), ref_in.grad) < 1e-3


def test_moe_experts_vs_loop():
    torch.manual_seed(6)
    n, k, E, H, I = 777, 4, 8, 256, 128
    x = bf(n, H).requires_grad_()
    w = torch.rand(n, k, device="cuda").requires_grad_()
    eids = torch.stack([torch.randperm(E, device="cuda")[:k] for _ in range(n)]).int()
    eids[::7, 0] = -1
    w1 = bf(E, 2 * I, H, scale=0.05)
    w2 = bf(E, H, I, scale=0.05)
    g1, g2 = torch.zeros_like(w1, dtype=torch.float32), torch.zeros_like(w2, dtype=torch.float32)
    ew = M.ExpertWeights(w1, w2, lambda: g1, lambda: g2)
    out = M.moe_experts(x, w, eids, ew)
    go = bf(n, H)
    out.backward(go)
    xr, wr = x.detach().float().requires_grad_(), w.detach().requires_grad_()
    w1r, w2r = w1.float().requires_grad_(), w2.float().requires_grad_()
    ref = M.moe_experts_ref(xr, wr, eids, w1r, w2r)
    ref.backward(go.float())
    _native.check_status()
    assert calc_diff(out.float(), ref) < 1e-3
    assert calc_diff(x.grad.float(), xr.grad) < 1e-3
    assert calc_diff(w.grad, wr.grad) < 1e-3
    assert calc_diff(g1, w1r.grad) < 1e-3
    assert calc_diff(g2, w2r.grad) < 1e-3


def test_moe_expert_wgrads_paired_across_micro_batches(monkeypatch):
    """With pairing on, three micro-batches (one pair + one flushed leftover) give the gradients of the unpaired path."""
    torch.manual_seed(16)
    k, E, H, I = 4, 8, 256, 128
    w1 = bf(E, 2 * I, H, scale=0.05)
    w2 = bf(E, H, I, scale=0.05)
    batches = []
    for n in (640, 333, 512):
        eids = torch.stack([torch.randperm(E, device="cuda")[:k] for _ in range(n)]).int()
        eids[::5, 1] = -1
        batches.append((bf(n, H), torch.rand(n, k, device="cuda"), eids, bf(n, H)))

    def run(paired):
        monkeypatch.setattr(M, "PAIR_EXPERT_WGRADS", paired)
        g1, g2 = torch.zeros_like(w1, dtype=torch.float32), torch.zeros_like(w2, dtype=torch.float32)
        dxs = []
        for x, w, eids, go in batches:
            x = x.clone().requires_grad_()
            ew = M.ExpertWeights(w1, w2, lambda: g1, lambda: g2)  # a new view per call, as the owning module makes
            M.moe_experts(x, w.clone().requires_grad_(), eids, ew).backward(go)
            dxs.append(x.grad)
        if paired:
            assert len(M._PENDING_WGRAD) == 1
        M.flush_pending_expert_wgrads()
        assert not M._PENDING_WGRAD
        _native.check_status()
        return g1, g2, dxs

    a1, a2, adx = run(False)
    b1, b2, bdx = run(True)
    assert calc_diff(a1, b1) < 1e-6 and calc_diff(a2, b2) < 1e-6
    for p, q in zip(adx, bdx):
        assert torch.equal(p, q)


@pytest.mark.parametrize("n,k,E,valid", [(2048, 8, 128, 1000), (700, 4, 16, 699), (64, 2, 8, 0)])
def test_route_sort_device_side_count(n, k, E, valid):
    """Slots at or past a device-side count are ignored (the fused EP transport sizes by capacity)."""
    torch.manual_seed(4)
    eids = torch.randint(0, E, (n, k), device="cuda", dtype=torch.int32)
    nv = torch.tensor([valid * k], device="cuda", dtype=torch.int32)
    offs, ros, sor = M.route_sort(eids, E, n_valid=nv)
    ref_in = eids.cpu().clone().view(-1)
    ref_in[valid * k:] = -1
    offs_r, ros_r, sor_r = M.route_sort_ref(ref_in, E, sor.numel())
    _native.check_status()
    assert torch.equal(offs.cpu(), offs_r) and torch.equal(ros.cpu(), ros_r)
    assert torch.equal(sor.cpu(), sor_r)


@pytest.mark.parametrize("causal,q_off,window", [(False, 0, None), (True, 0, None), (True, 256, 300), (True, 0, 100)])
def test_ring_blocks_kernel_vs_math(causal, q_off, window):
    """The kernel block path of ring attention (with a *global* lse in the backward) equals the fp32 math."""
    from pithtrain_b200.ops import attention_native as N
    from pithtrain_b200.ops import ring_attention as R

    torch.manual_seed(11)
    B, S, Hq, Hkv, D = 2, 256, 8, 2, 64
    q, k, v = bf(B, S, Hq, D), bf(B, S, Hkv, D), bf(B, S, Hkv, D)
    do = bf(B, S, Hq, D)
    outs = []
    for own in (True, False):
        N.ENABLED = own
        try:
            o, lse = R.block_fwd(q, k, v, D ** -0.5, causal, q_off, window)
            # a larger global lse, as when other blocks contributed too
            lse_g = lse + 0.3
            o_g = o.float() * torch.exp(lse - lse_g).permute(0, 2, 1).unsqueeze(-1)
            grads = R.block_bwd(do, q, k, v, o_g, lse_g, D ** -0.5, causal, q_off, window)
            outs.append((o, lse) + tuple(grads))
        finally:
            N.ENABLED = True
    _native.check_status()
    for a, b in zip(*outs):
        assert a.shape == b.shape
        fin = torch.isfinite(b.float())
        assert calc_diff(a.float()[fin], b.float()[fin]) < 3e-4


def test_bounded_wait_reports_through_status_word():
    """A wait on a flag that nothing sets gives up after its time limit, records the reason in the status word and
    leaves the context usable (the host learns of the failure, no kernel spins forever)."""
    import time

    ctl = torch.zeros(128, dtype=torch.int32, device="cuda")
    torch.cuda.synchronize()
    _native.set_peer_wait_limit(0.5)  # the run-time limit of waits on a peer's flag
    try:
        t0 = time.time()
        rc = _native.lib().pt_symm_wait(ctl.data_ptr(), 0, 1, 1, _native.stream_ptr())
        assert rc == 0
        torch.cuda.synchronize()
        waited = time.time() - t0
        assert 0.3 < waited < 5.0, waited
        with pytest.raises(RuntimeError, match="4|peer|timeout"):
            _native.check_status()
        _native.check_status()  # cleared by the read
        y = bf(64, 64) + 1  # the context still works
        assert torch.isfinite(y.float()).all()
    finally:
        _native.set_peer_wait_limit(2.0)


def test_train_step_status_check_raises_after_a_timed_out_wait():
    """What the train step does once per step: read the status word and raise on every rank if a wait ran out."""
    from pithtrain_b200.tasks.pretrain_lm import raise_on_kernel_status, read_kernel_status

    ctl = torch.zeros(128, dtype=torch.int32, device="cuda")
    _native.set_peer_wait_limit(0.2)
    try:
        assert _native.lib().pt_symm_wait(ctl.data_ptr(), 0, 1, 1, _native.stream_ptr()) == 0
        torch.cuda.synchronize()
        status = read_kernel_status()
        assert status == 4
        with pytest.raises(_native.KernelStatusError, match="peer"):
            raise_on_kernel_status(status, status)
        assert read_kernel_status() == 0  # cleared by the read
        raise_on_kernel_status(0, 0)      # a clean step passes
    finally:
        _native.set_peer_wait_limit(2.0)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_accumulate_colsum_into_main_grad(dtype):
    from pithtrain_b200.ops.common import accumulate_colsum

    torch.manual_seed(12)
    part = torch.randn(300, 256, device="cuda")
    p = torch.nn.Parameter(torch.zeros(128, device="cuda", dtype=torch.bfloat16))
    p.main_grad = torch.randn(128, device="cuda").to(dtype)
    want = (p.main_grad.float() + part[:, 128:256].sum(0)).to(dtype)
    accumulate_colsum(p, part, 128, 256)
    _native.check_status()
    assert torch.allclose(p.main_grad.float(), want.float(), atol=1e-2 if dtype == torch.bfloat16 else 1e-4, rtol=1e-2)
    q = torch.nn.Parameter(torch.zeros(256, device="cuda", dtype=torch.bfloat16))  # no flat buffer: plain .grad
    accumulate_colsum(q, part)
    assert torch.allclose(q.grad.float(), part.sum(0), atol=0.2, rtol=2e-2)


def test_attention_sinks_and_packed_paths_on_gpu():
    """Sinks, packed sequences and sliding windows through the public entry point."""
    from pithtrain_b200.ops import attention as A

    torch.manual_seed(13)
    B, S, Hq, Hkv, D = 2, 512, 8, 2, 64
    q, k, v = [bf(B, S, h, D).requires_grad_() for h in (Hq, Hkv, Hkv)]
    sinks = torch.randn(Hq, device="cuda", requires_grad=True)
    go = bf(B, S, Hq, D)
    out = A.attention(q, k, v, True, None, None, sinks, None)
    got = (out,) + torch.autograd.grad(out, [q, k, v, sinks], go)
    ref = A.attention_ref(q, k, v, True, None, None, sinks, None)
    want = (ref,) + torch.autograd.grad(ref, [q, k, v, sinks], go)
    for a, b in zip(got, want):
        assert calc_diff(a.float(), b.float()) < 5e-4
    cu = torch.tensor([0, 100, 300, S], dtype=torch.int32, device="cuda")
    out = A.attention(q, k, v, True, None, None, None, cu)
    ref = A.attention_ref(q, k, v, True, None, None, None, cu)
    assert calc_diff(out.float(), ref.float()) < 3e-4
    out = A.attention(q, k, v, True, None, 127, sinks, None)  # GPT-OSS sliding-window layer: blocked form
    ref = A.attention_ref(q, k, v, True, None, 127, sinks, None)
    assert calc_diff(out.float(), ref.float()) < 3e-4


@pytest.mark.skipif(os.environ.get("PITHTRAIN_NS_GEMM", "library") != "own",
                    reason="Newton-Schulz on the own grouped GEMMs runs only with PITHTRAIN_NS_GEMM=own until it is timed")
@pytest.mark.parametrize("shape", [(8, 768, 2048), (4, 2048, 768), (1, 512, 2048), (2048, 4096)])
def test_newton_schulz_on_own_gemms_matches_library_products(shape):
    from pithtrain_b200.modules.optimizer import newtonschulz5_own_gemm

    torch.manual_seed(12)
    G = torch.randn(*shape, device="cuda").bfloat16()
    got = newtonschulz5_own_gemm(G).float()
    torch.cuda.synchronize()
    _native.check_status()
    os.environ["PITHTRAIN_NS_GEMM"] = "library"
    try:
        from pithtrain_b200.modules.optimizer import zeropower_via_newtonschulz5

        want = zeropower_via_newtonschulz5(G).float()
    finally:
        os.environ["PITHTRAIN_NS_GEMM"] = "own"
    assert got.shape == want.shape
    assert float((got - want).norm() / want.norm()) < 0.05


@pytest.mark.parametrize("E,H", [(4, 256), (32, 2880), (1, 64)])
def test_indexed_bias_add_and_segment_sum_kernels(E, H):
    """Per-expert bias on expert-sorted rows and its segmented gradient against plain tensor ops."""
    from pithtrain_b200.ops import moe as M
    from pithtrain_b200.ops.activations import indexed_bias_add

    torch.manual_seed(31)
    sizes = torch.randint(0, 70, (E,))
    sizes[0] = 0 if E > 1 else 40                       # an empty group must work
    offs = torch.cat([torch.zeros(1, dtype=torch.long), torch.cumsum(((sizes + 15) // 16) * 16, 0)]).int().cuda()
    R = int(offs[-1]) + 32                              # rows past offs[E] belong to no group
    x = bf(R, H, scale=1.0)
    bias = torch.nn.Parameter(bf(E, H, scale=1.0))
    gid = M.rows_group_id(offs, R).clamp(max=E - 1)
    n_rows = offs[E:E + 1]
    got = M.indexed_bias_add_rows(x, bias.detach(), offs, n_rows)
    want = x + bias.detach()[gid]
    last = int(offs[-1])
    assert torch.equal(got[:last], want[:last])
    # segmented sums, plain and row-weighted, bf16 and fp32 inputs
    w = torch.rand(R, device="cuda")
    o = offs.long()
    for src in (x, x.float()):
        for rw in (None, w):
            s = M.segment_sum(src, offs, E, row_w=rw)
            xf = src.float() if rw is None else src.float() * rw[:, None]
            ref = torch.stack([xf[o[g]:o[g + 1]].sum(0) for g in range(E)])
            assert torch.allclose(s, ref, atol=2e-3, rtol=1e-4)
    # the autograd op: bias gradient = per-group row sum of the incoming gradient
    xg = x[:last].clone().requires_grad_()
    y = indexed_bias_add(xg, bias, offs)
    go = bf(last, H, scale=1.0)
    y.backward(go)
    _native.check_status()
    ref_b = torch.stack([go.float()[o[g]:o[g + 1]].sum(0) for g in range(E)])
    grad = bias.grad if bias.grad is not None else bias.main_grad
    assert torch.allclose(grad.float(), ref_b, atol=0.3, rtol=2e-2)
    assert torch.equal(xg.grad, go)


@pytest.mark.parametrize("B,S,H,dk,dv", [(1, 256, 4, 128, 128), (2, 200, 2, 64, 64), (1, 1024, 8, 128, 128)])
def test_gated_delta_rule_recurrence_kernels(B, S, H, dk, dv):
    """The chunk-to-chunk pass of the gated delta rule on the kernels of csrc/gdr.cu (forward and backward) against the
    same pass in tensor ops, and the whole op against the token-by-token recurrence."""
    from pithtrain_b200.ops import gated_delta_rule as GD

    torch.manual_seed(41)
    N, C = (S + 63) // 64, 64
    mk = lambda *s: (torch.randn(*s, device="cuda") * 0.05).requires_grad_()  # small: the state must not blow up over N chunks
    w, qg, kd = mk(B, H, N, C, dk), mk(B, H, N, C, dk), mk(B, H, N, C, dk)
    u = mk(B, H, N, C, dv)
    a = (torch.rand(B, H, N, device="cuda") * 0.5 + 0.5).requires_grad_()
    go_v, go_o = torch.randn(B, H, N, C, dv, device="cuda"), torch.randn(B, H, N, C, dv, device="cuda")
    outs = []
    for fn in (GD._ChunkState.apply, GD._chunk_state_math):
        v_new, o_inter = fn(w, u, qg, kd, a)
        grads = torch.autograd.grad((v_new, o_inter), [w, u, qg, kd, a], (go_v, go_o))
        outs.append((v_new, o_inter) + grads)
    _native.check_status()
    for x, y in zip(*outs):
        assert calc_diff(x, y) < 1e-6, calc_diff(x, y)
    # the whole op in bf16 against the recurrence
    q, k = bf(B, S, H, dk, scale=1.0), torch.nn.functional.normalize(torch.randn(B, S, H, dk, device="cuda"), dim=-1).bfloat16()
    v = bf(B, S, H, dv, scale=1.0)
    g = -torch.rand(B, S, H, device="cuda") * 0.2
    beta = torch.rand(B, S, H, device="cuda")
    got = GD.gated_delta_rule(q, k, v, g, beta)
    ref = GD.gated_delta_rule_recurrent(q, k, v, g, beta)
    assert calc_diff(got.float(), ref.float()) < 1e-3


@pytest.mark.parametrize("B,S,H,D,dtype", [(1, 256, 8, 128, torch.bfloat16), (2, 96, 4, 64, torch.float32),
                                           (1, 40, 3, 192, torch.bfloat16)])
def test_merge_partial_kernel_vs_math(B, S, H, D, dtype):
    """The ring-attention merge kernel equals its fp32 tensor restatement, rows without any key so far included."""
    from pithtrain_b200.ops import ring_attention as R

    torch.manual_seed(21)
    out = torch.randn(B, S, H, D, device="cuda")
    lse = torch.randn(B, H, S, device="cuda") * 3
    # the partial as a slice of a wider buffer (row pitch larger than H * D), as the fused projections produce it
    wide = torch.randn(B, S, H * D + 64, device="cuda").to(dtype)
    o_p = wide[..., :H * D].view(B, S, H, D)
    lse_p = torch.randn(B, H, S, device="cuda") * 3
    lse[:, 0, :7] = float("-inf")            # nothing seen before
    lse_p[:, 1, 3:9] = float("-inf")         # nothing in this block
    lse[:, 2, 5] = float("-inf"); lse_p[:, 2, 5] = float("-inf")  # nothing at all
    out[:, :7, 0] = 0.0
    out[:, 5, 2] = 0.0
    ref_out, ref_lse = R.merge_partial_math(out.clone(), lse.clone(), o_p, lse_p)
    got_out, got_lse = R.merge_partial(out.clone(), lse.clone(), o_p, lse_p)
    _native.check_status()
    assert torch.equal(torch.isinf(got_lse), torch.isinf(ref_lse))
    fin = ~torch.isinf(ref_lse)
    assert (got_lse[fin] - ref_lse[fin]).abs().max() < 1e-4
    assert calc_diff(got_out, ref_out) < 1e-6
    assert float(got_out[:, 5, 2].abs().max()) == 0.0
