"""Worker: shard-group collectives over peer memory must match the NCCL reduce-scatter / all-gather."""
from __future__ import annotations

from types import SimpleNamespace

import torch
import torch.distributed as dist
import torch.nn as nn


def run(rank: int, world: int, grad_dtype_name: str, rounds: int = 3):
    from pithtrain_b200 import _native
    from pithtrain_b200.contexts import distributed
    from pithtrain_b200.modules.distributed import DistributedCfg, setup_distributed
    from pithtrain_b200.parallel.flat_shard import FlatShardGroup

    cfg = SimpleNamespace(distributed=DistributedCfg())
    setup_distributed(cfg, failfast=False)
    dev = distributed.device
    gdt = torch.float32 if grad_dtype_name == "fp32" else torch.bfloat16
    shapes = [(512, 384), (1000, 72), (256,), (3, 128, 64), (77, 8)]
    groups = []
    for fused in (True, False):
        torch.manual_seed(0)
        named = [(f"p{i}", nn.Parameter(torch.randn(*s, device=dev).bfloat16())) for i, s in enumerate(shapes)]
        g = FlatShardGroup("t", named, [], dist.group.WORLD, world, rank, gdt, device=dev, fused_collectives=fused)
        groups.append(g)
    fused, base = groups
    assert fused.comm is not None and base.comm is None
    assert torch.equal(fused.flat_param, base.flat_param)
    for it in range(rounds):
        gen = torch.Generator(device="cpu").manual_seed(1000 * it + rank)
        noise = torch.randn(fused.flat_grad.numel(), generator=gen).to(dev)
        for g in groups:
            g.flat_grad.copy_(noise.to(gdt))
            g.scale_grads(0.5)
            g.reduce_grads()
        a, b = fused.my_slice(fused.flat_grad).float(), base.my_slice(base.flat_grad).float()
        tol = 1e-6 if gdt == torch.float32 else 2e-2
        assert torch.allclose(a, b, atol=tol, rtol=tol), float((a - b).abs().max())
        sa, sb = fused.owned_grad_sumsq(), base.owned_grad_sumsq()
        assert abs(float(sa) - float(sb)) <= 2e-3 * abs(float(sb)) + 1e-6, (float(sa), float(sb))
        for g in groups:
            g.my_slice(g.flat_param).add_(0.25 * (rank + 1) + it)
            g.gather_params()
        for g in groups:
            g.wait_params()
            g.zero_grad()
        torch.cuda.synchronize()
        _native.check_status()
        assert torch.equal(fused.flat_param, base.flat_param), it
        assert float(fused.flat_grad.abs().max()) == 0.0
    dist.barrier()
    fused.comm.close()
