"""Shard-group collectives, bucket sweep: kernels over peer memory against NCCL reduce-scatter / all-gather.

    python -m torch.distributed.run --nproc-per-node 4 --master-addr 127.0.0.1 benchmarks/operators/bench_shard_collectives.py

For flat groups of 16 MB to 1 GB (bf16 parameters and bf16 gradient accumulators) it times, on the device with CUDA
events and as the max over ranks, (a) the gradient reduce-scatter with averaging and the sum-of-squares partials of
the gradient norm, and (b) the publication of the updated parameter regions to all ranks. Per-GPU link traffic of
either step is ``(W-1)/W`` of the group's bytes in one direction, so the roofline is that over the measured 770 GB/s
peer-copy bandwidth. Sizes below the 126 MB L2 are marked: part of their traffic never reaches HBM on the reading
side, so their figures say more about launch and flag latency than about bandwidth.
"""

import argparse
import os
import sys
from pathlib import Path
from types import SimpleNamespace

import torch
import torch.distributed as dist
import torch.nn as nn

sys.path.insert(0, str(Path(__file__).resolve().parents[2]))

LINK_GBS = 770.0
L2_BYTES = 126 << 20


def time_group(g, iters: int, warmup: int, dev):
    red, pub = [], []
    for it in range(iters + warmup):
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
        if it >= warmup:
            red.append(e[0].elapsed_time(e[1]))
            pub.append(e[1].elapsed_time(e[2]))
    t = torch.tensor([sorted(red)[len(red) // 2], sorted(pub)[len(pub) // 2]], device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t[0]), float(t[1])


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--sizes-mb", default="16,64,256,1024")
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    a = ap.parse_args()
    from pithtrain_b200 import _native
    from pithtrain_b200.contexts import distributed
    from pithtrain_b200.modules.distributed import DistributedCfg, setup_distributed
    from pithtrain_b200.parallel.flat_shard import FlatShardGroup

    cfg = SimpleNamespace(distributed=DistributedCfg())
    setup_distributed(cfg, failfast=False)
    W, rank, dev = int(os.environ.get("WORLD_SIZE", "1")), distributed.rank, distributed.device
    if W < 2:
        raise SystemExit("needs at least 2 ranks")
    for mb in (int(x) for x in a.sizes_mb.split(",")):
        total = mb << 20  # bytes of bf16 parameters in the group
        per = total // 2 // (2 * W)  # 2W equal parameters so that every owner holds the same amount
        row = {}
        for fused in (True, False):
            named = [(f"w{i}", nn.Parameter(torch.zeros(per, device=dev, dtype=torch.bfloat16))) for i in range(2 * W)]
            g = FlatShardGroup("bw", named, [], dist.group.WORLD, W, rank, torch.bfloat16, device=dev, fused_collectives=fused)
            row["fused" if fused else "nccl"] = time_group(g, a.iters, a.warmup, dev)
            if g.comm is not None:
                g.comm.close()
            del g, named
            torch.cuda.empty_cache()
        _native.check_status()
        if rank == 0:
            link_bytes = (W - 1) / W * total
            floor = link_bytes / (LINK_GBS * 1e9) * 1e3
            note = "  (< L2)" if total < L2_BYTES else ""
            for name, (r, p) in row.items():
                print(f"{mb:>5d} MB W={W} {name:<5s}: reduce-scatter {r:.3f} ms ({link_bytes / r / 1e6:.0f} GB/s, {floor / r:.2f} of link "
                      f"roofline), publish {p:.3f} ms ({link_bytes / p / 1e6:.0f} GB/s, {floor / p:.2f}){note}", flush=True)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
