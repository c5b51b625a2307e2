"""Worker: zigzag ring attention vs dense attention over the full sequence (outputs and all gradients)."""
from __future__ import annotations

from types import SimpleNamespace

import torch
import torch.distributed as dist


def zigzag_slice(x, cp, r, dim=1):
    S = x.shape[dim]
    b = S // (2 * cp)
    return torch.cat([x.narrow(dim, r * b, b), x.narrow(dim, (2 * cp - 1 - r) * b, b)], dim=dim)


def run(rank, world, case, device_type="cpu", rounds=1):
    """``rounds`` > 2 exercises the slot reuse of the peer-memory transport on GPUs."""
    for it in range(rounds):
        _run_once(rank, world, case, device_type, first=(it == 0), seed=3 + it)
    if device_type == "cuda":
        from pithtrain_b200 import _native

        torch.cuda.synchronize()
        _native.check_status()


def _run_once(rank, world, case, device_type, first, seed):
    from pithtrain_b200.contexts import distributed
    from pithtrain_b200.modules.distributed import DistributedCfg, setup_distributed
    from pithtrain_b200.ops.attention import attention_ref
    from pithtrain_b200.ops.ring_attention import mla_ring_attention_func, ring_attention_func
    from utilities import calc_diff

    if first:
        cfg = SimpleNamespace(distributed=DistributedCfg())
        cfg.distributed.context_parallel_size = world
        setup_distributed(cfg, failfast=False)
    cp, r = world, distributed.cp_rank
    torch.manual_seed(seed)
    if device_type == "cuda":
        torch.set_default_device(distributed.device)
        torch.backends.cuda.matmul.allow_tf32 = False  # the oracle comparison wants real fp32 products
    tol = 1e-9 if device_type == "cpu" else 1e-5  # TF32-free fp32 on the GPU, different reduction order
    B, S = 2, 16 * cp
    if case == "mla":
        H, nope, rope, vd, lat = 3, 8, 4, 6, 10
        q_nope, q_pe = torch.randn(B, S, H, nope), torch.randn(B, S, H, rope)
        nkv, k_pe = torch.randn(B, S, lat), torch.randn(B, S, 1, rope)
        W = torch.randn(H * (nope + vd), lat) * 0.3
        go = torch.randn(B, S, H, vd)
        scale = (nope + rope) ** -0.5
        # dense oracle
        leaves = [t.clone().requires_grad_() for t in (q_nope, q_pe, nkv, k_pe, W)]
        kv = torch.nn.functional.linear(leaves[2], leaves[4]).view(B, S, H, nope + vd)
        k = torch.cat([kv[..., :nope], leaves[3].expand(-1, -1, H, -1)], -1)
        ref = attention_ref(torch.cat([leaves[0], leaves[1]], -1), k, kv[..., nope:], causal=True, scale=scale)
        ref.backward(go)
        mine = [zigzag_slice(t, cp, r).clone().requires_grad_() for t in (q_nope, q_pe, nkv, k_pe)]
        Wp = torch.nn.Parameter(W.clone())
        out = mla_ring_attention_func(mine[0], mine[1], mine[2], mine[3], Wp, scale, nope, vd)
        out.backward(zigzag_slice(go, cp, r))
        assert calc_diff(out, zigzag_slice(ref.detach(), cp, r)) < tol
        for a, b in zip(mine, leaves[:4]):
            assert calc_diff(a.grad, zigzag_slice(b.grad, cp, r)) < tol
        gW = Wp.grad.clone()
        dist.all_reduce(gW, group=distributed.cp_group)
        assert calc_diff(gW, leaves[4].grad) < tol
        return
    Hq, Hkv, D = (4, 2, 8) if case != "mha" else (2, 2, 8)
    window = 5 if case == "window_sink" else None
    if case == "gqa_d128_bf16":
        # the shape family of the tcgen05 attention kernel: one sequence, head dim 128, blocks of 128 tokens, bf16
        B, S, Hq, Hkv, D = 1, 256 * cp, 4, 2, 128
        tol = 3e-3 if device_type == "cuda" else 1e-4
        mk = lambda *shape: torch.randn(*shape).bfloat16()  # noqa: E731
        q, k, v, go = mk(B, S, Hq, D), mk(B, S, Hkv, D), mk(B, S, Hkv, D), mk(B, S, Hq, D)
        leaves = [t.float().requires_grad_() for t in (q, k, v)]
        ref = attention_ref(leaves[0], leaves[1], leaves[2], causal=True)
        ref.backward(go.float())
        mine = [zigzag_slice(t, cp, r).clone().requires_grad_() for t in (q, k, v)]
        out = ring_attention_func(mine[0], mine[1], mine[2])
        out.backward(zigzag_slice(go, cp, r))
        assert calc_diff(out.float(), zigzag_slice(ref.detach(), cp, r)) < tol
        for a, b in zip(mine, leaves):
            assert calc_diff(a.grad.float(), zigzag_slice(b.grad, cp, r)) < tol
        return
    q, k, v = torch.randn(B, S, Hq, D), torch.randn(B, S, Hkv, D), torch.randn(B, S, Hkv, D)
    sinks = torch.randn(Hq) if case == "window_sink" else None
    go = torch.randn(B, S, Hq, D)
    leaves = [t.clone().requires_grad_() for t in (q, k, v)] + ([sinks.clone().requires_grad_()] if sinks is not None else [])
    ref = attention_ref(leaves[0], leaves[1], leaves[2], causal=True, window_left=window,
                        sinks=leaves[3] if sinks is not None else None)
    ref.backward(go)
    mine = [zigzag_slice(t, cp, r).clone().requires_grad_() for t in (q, k, v)]
    sp = torch.nn.Parameter(sinks.clone()) if sinks is not None else None
    out = ring_attention_func(mine[0], mine[1], mine[2], window_left=window, sinks=sp)
    out.backward(zigzag_slice(go, cp, r))
    assert calc_diff(out, zigzag_slice(ref.detach(), cp, r)) < tol, calc_diff(out, zigzag_slice(ref.detach(), cp, r))
    for a, b in zip(mine, leaves[:3]):
        assert calc_diff(a.grad, zigzag_slice(b.grad, cp, r)) < tol
    if sinks is not None:
        gs = sp.grad.clone()
        dist.all_reduce(gs, group=distributed.cp_group)
        assert calc_diff(gs, leaves[3].grad) < 10 * tol
