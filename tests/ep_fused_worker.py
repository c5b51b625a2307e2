"""Worker: the peer-memory exchange must reproduce the all-to-all exchange, forward and backward."""
from __future__ import annotations

from types import SimpleNamespace

import torch
import torch.distributed as dist


def run(rank: int, world: int, m: int, H: int, E: int, k: int, rounds: int = 3):
    from pithtrain_b200 import _native
    from pithtrain_b200.contexts import distributed
    from pithtrain_b200.modules.distributed import DistributedCfg, setup_distributed
    from pithtrain_b200.parallel.ep import CollectiveExchange, home_reduce
    from pithtrain_b200.parallel.ep_fused import FusedExchange

    cfg = SimpleNamespace(distributed=DistributedCfg())
    cfg.distributed.expert_parallel_size = world
    setup_distributed(cfg, failfast=False)
    dev = distributed.device
    base = CollectiveExchange(distributed.ep_group, world, rank)
    fused = FusedExchange(distributed.ep_group, world, rank)
    g = torch.Generator(device="cpu").manual_seed(100 + rank)
    for it in range(rounds):
        x0 = torch.randn(m, H, generator=g).to(dev).bfloat16()
        w0 = torch.rand(m, k, generator=g).to(dev)
        if it == rounds - 1 and E // world >= k:
            # collapsed router: every token of every rank goes to rank 0's experts (the exact worst case, ep * m rows)
            idx = torch.stack([torch.randperm(E // world, generator=g)[:k] for _ in range(m)]).int().to(dev)
        else:
            idx = torch.stack([torch.randperm(E, generator=g)[:k] for _ in range(m)]).int().to(dev)
        outs = []
        for ex in (base, fused):
            x, w = x0.clone().requires_grad_(), w0.clone().requires_grad_()
            plan = ex.plan(idx, E)
            rx, rw = ex.dispatch(x, w, plan)
            n = plan.n_recv if plan.n_recv_dev is None else int(plan.n_recv_dev)
            eids = plan.recv_eids[:n]
            # a stand-in for the expert block: depends on rows, weights and local expert ids
            valid = (eids >= 0).float()
            partial = rx[:n].float() * ((rw[:n] * valid * (eids.float() + 2)).sum(-1, keepdim=True))
            if rx.shape[0] > n:
                partial = torch.cat([partial, rx[n:].float() * 0])
            back = ex.combine(partial.to(x.dtype), plan)
            out = back if getattr(plan, "reduced", False) else home_reduce(back, plan)
            go = torch.randn(m, H, generator=torch.Generator().manual_seed(7 + it)).to(dev).bfloat16()
            out.backward(go)
            torch.cuda.synchronize()
            # canonical receive order differs between transports; compare order-free quantities
            outs.append((out.detach().float(), x.grad.float(), w.grad.float(), n,
                         rx[:n].float().sum(0), (eids >= 0).sum()))
        _native.check_status()
        (o1, gx1, gw1, n1, s1, c1), (o2, gx2, gw2, n2, s2, c2) = outs
        assert n1 == n2 and int(c1) == int(c2), (n1, n2)
        assert torch.allclose(s1, s2, atol=0.5, rtol=2e-2)
        assert torch.allclose(o1, o2, atol=2e-2, rtol=2e-2), float((o1 - o2).abs().max())
        assert torch.allclose(gx1, gx2, atol=5e-2, rtol=2e-2), float((gx1 - gx2).abs().max())
        assert torch.allclose(gw1, gw2, atol=5e-1, rtol=3e-2), float((gw1 - gw2).abs().max())
    dist.barrier()
    fused.close()


def run_checked(rank: int, world: int, m: int, H: int, E: int, k: int):
    """Bounds-checking build of the library: a corrupted send plan (a token index one past the micro-batch) is
    recorded in the status word and the row is skipped, instead of a read outside the activations and a store of
    garbage into the peer's partition."""
    import os

    os.environ["PITHTRAIN_CHECKED_LIB"] = "1"
    from pithtrain_b200 import _native
    from pithtrain_b200.contexts import distributed
    from pithtrain_b200.modules.distributed import DistributedCfg, setup_distributed
    from pithtrain_b200.parallel.ep_fused import FusedExchange

    assert _native._LIB_PATH.name == "libpithb200_checked.so", _native._LIB_PATH
    cfg = SimpleNamespace(distributed=DistributedCfg())
    cfg.distributed.expert_parallel_size = world
    setup_distributed(cfg, failfast=False)
    dev = distributed.device
    fused = FusedExchange(distributed.ep_group, world, rank)
    g = torch.Generator(device="cpu").manual_seed(200 + rank)
    x = torch.randn(m, H, generator=g).to(dev).bfloat16()
    w = torch.rand(m, k, generator=g).to(dev)
    idx = torch.stack([torch.randperm(E, generator=g)[:k] for _ in range(m)]).int().to(dev)
    plan = fused.plan(idx, E)
    rx, _ = fused.dispatch(x, w, plan)      # a clean exchange first
    torch.cuda.synchronize()
    assert _native.fetch_status() == 0
    plan = fused.plan(idx, E)
    plan.send_token_idx[0] = m              # one past the last token
    fused.dispatch(x, w, plan)
    torch.cuda.synchronize()
    assert _native.fetch_status() == 8      # PT_ERR_BOUNDS
    dist.barrier()
    fused.close()
