"""Worker: reference-named communication helper on gloo ranks."""
import torch
import torch.distributed as dist


def run_all_to_all(rank: int, world: int):
    from pithtrain.operators.all_to_all import direct_all_to_all  # through the reference's package name

    dist.init_process_group("gloo", rank=rank, world_size=world)
    send_counts = [1 + ((rank + d) % 3) for d in range(world)]
    recv_counts = [1 + ((s + rank) % 3) for s in range(world)]
    x = torch.cat([torch.full((c, 4), float(10 * rank + d)) for d, c in enumerate(send_counts)])
    out = direct_all_to_all(x, recv_counts, send_counts, dist.group.WORLD)
    out.comm_work.wait()
    want = torch.cat([torch.full((c, 4), float(10 * s + rank)) for s, c in enumerate(recv_counts)])
    assert torch.equal(out, want), (out, want)
    dist.destroy_process_group()
