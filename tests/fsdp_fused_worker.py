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
    # guard words behind every symmetric allocation: intact after the exchanges, and a write behind the buffer (what an
    # out-of-range peer store would do; made from the host side here) is reported with the buffer's name
    from pithtrain_b200.parallel.symm_mem import GuardOverrun, check_all_guards

    check_all_guards()
    saved = int(fused.comm.grad_buf._guard[3])
    fused.comm.grad_buf._guard[3] = 0
    try:
        check_all_guards()
    except GuardOverrun as e:
        assert "shard gradients" in str(e), str(e)
    else:
        raise AssertionError("an overwritten guard word went unnoticed")
    fused.comm.grad_buf._guard[3] = saved
    dist.barrier()
    fused.comm.close()
    if rounds >= 3 and gdt == torch.bfloat16:
        _report_bandwidth(rank, world, dev)


def _report_bandwidth(rank: int, world: int, dev) -> None:
    """Device-timed reduce-scatter and parameter publication of a 512 MB group (printed by rank 0)."""
    from pithtrain_b200.parallel.flat_shard import FlatShardGroup

    p = nn.Parameter(torch.zeros(world * 64 * 1024 * 1024 // world, device=dev, dtype=torch.bfloat16))
    named = [(f"w{i}", nn.Parameter(torch.zeros(32 * 1024 * 1024, device=dev, dtype=torch.bfloat16))) for i in range(2 * world)]
    g = FlatShardGroup("bw", named, [], dist.group.WORLD, world, rank, torch.bfloat16, device=dev, fused_collectives=True)
    del p
    region_bytes = g.region * 2
    times = {"reduce": [], "push": []}
    for it in range(6):
        g.flat_grad.fill_(0.5)
        dist.barrier()
        e = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
        e[0].record()
        g.reduce_grads()
        e[1].record()
        g.gather_params()
        g.wait_params()
        e[2].record()
        g.zero_grad()
        torch.cuda.synchronize()
        if it >= 2:
            times["reduce"].append(e[0].elapsed_time(e[1]))
            times["push"].append(e[1].elapsed_time(e[2]))
    t = torch.tensor([min(times["reduce"]), min(times["push"])], device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    if rank == 0:
        remote = (world - 1) * region_bytes
        print(f"[fsdp-fused bandwidth] W={world} region {region_bytes / 2**20:.0f} MiB: reduce-scatter {float(t[0]):.3f} ms "
              f"({remote / float(t[0]) / 1e6:.0f} GB/s pulled per GPU), publish {float(t[1]):.3f} ms "
              f"({remote / float(t[1]) / 1e6:.0f} GB/s pushed per GPU); measured peer copy 770 GB/s per direction", flush=True)
    dist.barrier()
    g.comm.close()
