"""Expert-parallel dispatch + combine round trip: fused peer-memory transport against NCCL all-to-all.

    python -m torch.distributed.run --nproc-per-node 4 --master-addr 127.0.0.1 benchmarks/operators/bench_ep_exchange.py

Per transport: milliseconds (CUDA events, max over ranks) of plan + dispatch + combine forward and of the
backward of both, for one micro-batch of ``--tokens`` rows of width ``--hidden`` routed top-``k`` over
``--experts`` experts, and the NVLink roofline: de-duplicated bytes leaving a GPU per direction divided by the
measured 770 GB/s peer-copy bandwidth. ``--routing`` selects uniform subsets, top-k of N(0,1) logits, or a
Zipf(1.2)-skewed expert popularity; ``--sweep`` runs 4096, 8192, 16384 and 32768 tokens per rank.
"""

import argparse
import os
import sys
from pathlib import Path
from types import SimpleNamespace

import torch
import torch.distributed as dist

sys.path.insert(0, str(Path(__file__).resolve().parents[2]))
from benchmarks.operators.utilities import make_routing, remote_rows_by_destination  # noqa: E402
from pithtrain_b200.parallel.ep import CollectiveExchange, home_reduce  # noqa: E402

LINK_GBS = 770.0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=4096)
    ap.add_argument("--hidden", type=int, default=2048)
    ap.add_argument("--experts", type=int, default=128)
    ap.add_argument("--k", type=int, default=8)
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--routing", choices=["uniform", "normal", "zipf"], default="uniform")
    ap.add_argument("--sweep", action="store_true", help="tokens per rank 4096 ... 32768 instead of --tokens")
    a = ap.parse_args()
    from pithtrain_b200.contexts import distributed
    from pithtrain_b200.modules.distributed import DistributedCfg, setup_distributed
    from pithtrain_b200.parallel.ep_fused import FusedExchange

    cfg = SimpleNamespace(distributed=DistributedCfg())
    cfg.distributed.expert_parallel_size = int(os.environ.get("WORLD_SIZE", "1"))
    setup_distributed(cfg, failfast=False)
    ep, rank, dev = distributed.ep_size, distributed.ep_rank, distributed.device
    transports = (("nccl all_to_all", CollectiveExchange(distributed.ep_group, ep, rank)),
                  ("fused peer-memory", FusedExchange(distributed.ep_group, ep, rank)))
    sizes = sorted((4096, 8192, 16384, 32768), reverse=True) if a.sweep else [a.tokens]  # largest first sizes the buffers once
    for m in sizes:
        run_case(a, m, transports, distributed)
    dist.barrier()
    dist.destroy_process_group()


def run_case(a, m, transports, distributed):
    ep, rank, dev = distributed.ep_size, distributed.ep_rank, distributed.device
    H, E, k = a.hidden, a.experts, a.k
    g = torch.Generator().manual_seed(rank)
    x0 = torch.randn(m, H, generator=g).to(dev).bfloat16()
    w0 = torch.rand(m, k, generator=g).to(dev)
    idx_cpu = make_routing(m, E, k, a.routing, seed=rank)
    idx = idx_cpu.to(dev)
    # the busiest link direction of any GPU sets the floor: rows it sends out, or rows it takes in (skewed routing)
    out_rows = remote_rows_by_destination(idx_cpu, E, ep, rank).float().to(dev)
    in_rows = out_rows.clone()
    dist.all_reduce(in_rows)  # element g: rows arriving at rank g from all other ranks
    busiest = torch.stack([out_rows.sum(), in_rows.max()]).max()
    dist.all_reduce(busiest, op=dist.ReduceOp.MAX)
    floor_ms = float(busiest) * H * 2 / (LINK_GBS * 1e9) * 1e3
    for name, ex in transports:
        fwd, bwd = [], []
        for it in range(a.iters + 5):
            x, w = x0.clone().requires_grad_(), w0.clone().requires_grad_()
            dist.barrier()
            e = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
            e[0].record()
            plan = ex.plan(idx, E)
            rx, rw = ex.dispatch(x, w, plan)
            back = ex.combine(rx * rw.sum(-1, keepdim=True).to(rx.dtype), plan)
            out = back if getattr(plan, "reduced", False) else home_reduce(back, plan)
            e[1].record()
            out.backward(x0)
            e[2].record()
            torch.cuda.synchronize()
            if it >= 5:
                fwd.append(e[0].elapsed_time(e[1]))
                bwd.append(e[1].elapsed_time(e[2]))
        t = torch.tensor([sorted(fwd)[len(fwd) // 2], sorted(bwd)[len(bwd) // 2]], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        if distributed.rank == 0:
            print(f"{name:<20s} ep={ep} tokens={m} H={H} top{k}/{E} {a.routing}: fwd {t[0]:.3f} ms, bwd {t[1]:.3f} ms; NVLink "
                  f"floor for the two transfers of one pass {2 * floor_ms:.3f} ms -> fwd at {2 * floor_ms / float(t[0]):.2f} "
                  f"of link roofline", flush=True)
    from pithtrain_b200 import _native

    _native.check_status()


if __name__ == "__main__":
    main()
