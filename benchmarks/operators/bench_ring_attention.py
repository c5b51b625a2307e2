"""Zigzag ring attention forward/backward time per context-parallel width.

    python -m torch.distributed.run --nproc-per-node 4 --master-addr 127.0.0.1 benchmarks/operators/bench_ring_attention.py --seq 32768

Every rank holds its two zigzag blocks of a ``--seq`` token sequence; times are CUDA-event medians, max over
ranks, after 10 warm-up iterations (the reference's harness: benchmarks/operators/bench_ring_attention.py:28,53-74,
25 warm-up and 100 timed iterations). Reports achieved TFLOP/s per GPU on the causal FLOP count.
"""

import argparse
import os
import sys
from pathlib import Path
from types import SimpleNamespace

import torch
import torch.distributed as dist

sys.path.insert(0, str(Path(__file__).resolve().parents[2]))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--seq", type=int, default=16384)
    ap.add_argument("--heads", type=int, default=32)
    ap.add_argument("--kv-heads", type=int, default=4)
    ap.add_argument("--head-dim", type=int, default=128)
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--iters", type=int, default=30)
    a = ap.parse_args()
    from pithtrain_b200.contexts import distributed
    from pithtrain_b200.modules.distributed import DistributedCfg, setup_distributed
    from pithtrain_b200.ops.ring_attention import ring_attention_func

    cfg = SimpleNamespace(distributed=DistributedCfg())
    cfg.distributed.context_parallel_size = int(os.environ.get("WORLD_SIZE", "1"))
    setup_distributed(cfg, failfast=False)
    cp, dev = distributed.cp_size, distributed.device
    S = a.seq // cp
    q = torch.randn(a.batch, S, a.heads, a.head_dim, device=dev, dtype=torch.bfloat16, requires_grad=True)
    k = torch.randn(a.batch, S, a.kv_heads, a.head_dim, device=dev, dtype=torch.bfloat16, requires_grad=True)
    v = torch.randn(a.batch, S, a.kv_heads, a.head_dim, device=dev, dtype=torch.bfloat16, requires_grad=True)
    go = torch.randn(a.batch, S, a.heads, a.head_dim, device=dev, dtype=torch.bfloat16)
    fwd, bwd = [], []
    for it in range(a.iters + 10):
        dist.barrier()
        e = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
        e[0].record()
        o = ring_attention_func(q, k, v)
        e[1].record()
        o.backward(go)
        e[2].record()
        torch.cuda.synchronize()
        q.grad = k.grad = v.grad = None
        if it >= 10:
            fwd.append(e[0].elapsed_time(e[1]))
            bwd.append(e[1].elapsed_time(e[2]))
    t = torch.tensor([sorted(fwd)[len(fwd) // 2], sorted(bwd)[len(bwd) // 2]], device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    flops = 4 * a.batch * a.seq * a.seq * a.heads * a.head_dim / 2 / cp  # causal, per GPU, forward
    if distributed.rank == 0:
        print(f"ring attention cp={cp} seq={a.seq} heads={a.heads}/{a.kv_heads} d={a.head_dim}: fwd {t[0]:.3f} ms "
              f"({flops / float(t[0]) / 1e9:.0f} TF/GPU), bwd {t[1]:.3f} ms ({2.5 * flops / float(t[1]) / 1e9:.0f} TF/GPU)", flush=True)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
