"""NVLink peer bandwidth through the framework's own copy kernel, against the runtime's peer copy.

    python -m torch.distributed.run --nproc-per-node 2 --master-addr 127.0.0.1 benchmarks/operators/bench_link.py

Every rank pulls `--mib` MiB from the next rank's symmetric buffer (loads over NVLink) and pushes the same amount
(stores over NVLink) with ``pt_symm_copy``; rank 0 prints GB/s per direction (CUDA events, max time over ranks)
next to the 770 GB/s per direction measured for a plain peer copy on this pool and the 900 GB/s nominal figure.
"""

import argparse
import sys
from pathlib import Path
from types import SimpleNamespace

import torch
import torch.distributed as dist

sys.path.insert(0, str(Path(__file__).resolve().parents[2]))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--mib", type=int, default=512)
    ap.add_argument("--iters", type=int, default=10)
    a = ap.parse_args()
    from pithtrain_b200 import _native
    from pithtrain_b200.contexts import distributed
    from pithtrain_b200.modules.distributed import DistributedCfg, setup_distributed
    from pithtrain_b200.parallel.symm_mem import SymmetricBuffer

    cfg = SimpleNamespace(distributed=DistributedCfg())
    setup_distributed(cfg, failfast=False)
    dev, rank, world = distributed.device, distributed.rank, distributed.world_size
    nbytes = a.mib << 20
    buf = SymmetricBuffer(nbytes, dist.group.WORLD, dev)
    local = torch.empty(nbytes, dtype=torch.uint8, device=dev)
    peer = buf.peer_ptrs[(rank + 1) % world]
    L = _native.lib()

    def timed(fn):
        times = []
        for it in range(a.iters + 3):
            dist.barrier()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            torch.cuda.synchronize()
            if it >= 3:
                times.append(e0.elapsed_time(e1))
        t = torch.tensor([sorted(times)[len(times) // 2]], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t)

    st = lambda: _native.stream_ptr()
    results = {}
    for ctas in (16, 32, 64, 148, 0):
        results[f"pull, {ctas or 'all'} CTAs"] = timed(lambda: _native.check(L.pt_symm_copy(local.data_ptr(), peer, nbytes, ctas, st()), "pt_symm_copy"))
    results["push, all CTAs"] = timed(lambda: _native.check(L.pt_symm_copy(peer, local.data_ptr(), nbytes, 0, st()), "pt_symm_copy"))
    results["local copy (HBM)"] = timed(lambda: _native.check(L.pt_symm_copy(local.data_ptr(), buf.local_ptr, nbytes, 0, st()), "pt_symm_copy"))
    if rank == 0:
        print(f"{world} GPUs, {a.mib} MiB per transfer, every rank transfers at once; reference: 770 GB/s measured peer copy, 900 nominal")
        for k, ms in results.items():
            print(f"  {k:<22s}{ms:8.3f} ms  {nbytes / ms / 1e6:8.1f} GB/s per direction")
    dist.barrier()
    buf.close()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
