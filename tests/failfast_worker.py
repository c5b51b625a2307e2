"""Worker for the failure-detection tests (CPU, gloo): one rank fails on the host, the others must notice."""
import os
import sys
import time
from datetime import timedelta
from types import SimpleNamespace

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main():
    mode = sys.argv[1]
    import torch
    import torch.distributed as dist

    from pithtrain_b200.modules.distributed import DistributedCfg, setup_distributed

    cfg = SimpleNamespace(distributed=DistributedCfg())
    cfg.distributed.timeout = timedelta(seconds=4)
    setup_distributed(cfg, failfast=True)
    rank = dist.get_rank()
    x = torch.ones(1)
    dist.all_reduce(x)  # everybody is up
    if mode == "raise":
        if rank == 1:
            raise RuntimeError("injected host-side failure on rank 1")
        dist.all_reduce(x)  # rank 1 never joins: must end with an error after the group timeout
        print("UNEXPECTED: collective completed", flush=True)
    elif mode == "never_joins":
        if rank == 1:
            time.sleep(30)  # alive but absent
            return
        dist.all_reduce(x)
        print("UNEXPECTED: collective completed", flush=True)
    elif mode == "thread":
        import threading

        if rank == 0:
            t = threading.Thread(target=lambda: (_ for _ in ()).throw(ValueError("injected failure in a helper thread")))
            t.start()
            t.join()
            time.sleep(30)  # the hook must have ended the process before this returns
        else:
            time.sleep(1)


if __name__ == "__main__":
    main()
