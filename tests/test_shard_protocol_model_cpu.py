"""Exhaustive interleaving check of the flag protocol of the shard-group collectives over peer memory
(``csrc/fsdp_fused.cu``, driven by ``parallel/fsdp_fused.py`` from ``tasks/pretrain_lm.py: forward_backward_update``).

Per optimizer step ``e`` every rank runs, in program order on one stream:

    forward / backward       reads every region of its parameter buffer, accumulates into every region of its gradients
    signal_ready(e)          release-stores READY[me] = e where the peers can see it
    reduce_scatter(e)        waits READY[p] >= e for every p, reads region `me` of every peer's gradient buffer,
                             release-stores ACK[me] = e ("done reading")
    optimizer                rewrites the owned parameter region
    push_params(e)           stores the owned region into every peer's parameter buffer, release-stores PUSHED[me] = e
    wait_params(e)           waits PUSHED[p] >= e for every p
    zero_grad                waits ACK[p] >= e for every p, then clears its gradient buffer

The ranks' streams interleave arbitrarily. The checker walks every reachable state and asserts that a gradient buffer is
never cleared or accumulated into while a peer still reads it for an earlier step, that a reduction reads only final
gradients of its own step, that a forward never reads a region whose update of the previous step has not arrived, and
that a peer's parameter store never lands while the target's forward / backward of an earlier step is still reading.
Each guard removed in turn must be caught.
"""
from collections import deque
from typing import List, Tuple

import pytest


class Race(Exception):
    pass


class Stuck(Exception):
    pass


def program(W: int, steps: int, *, wait_ready: bool = True, wait_acks: bool = True, wait_params: bool = True,
            ready_after_backward: bool = True, zero_before_push: bool = False) -> List[Tuple]:
    prog: List[Tuple] = []
    for e in range(1, steps + 1):
        if not ready_after_backward:
            prog.append(("ready", e))
        prog += [("fwd_begin", e), ("fwd_end", e)]
        if ready_after_backward:
            prog.append(("ready", e))
        if wait_ready:
            prog.append(("wait_ready", e))
        prog += [("reduce_begin", e), ("reduce_end", e), ("ack", e), ("optimizer", e)]
        clear = ([("wait_acks", e)] if wait_acks else []) + [("zero", e)]
        if zero_before_push:
            prog += clear  # a caller that clears its gradients right after the optimizer step
        prog += [("push", e), ("pushed", e)]
        if wait_params:
            prog.append(("wait_params", e))
        if not zero_before_push:
            prog += clear
    return prog


def explore(W: int, steps: int, **mut) -> int:
    prog = program(W, steps, **mut)
    n = len(prog)
    start = tuple([0] * W)
    seen = {start}
    queue = deque([start])

    def value(rank_pc: int, kind: str) -> int:
        """Largest epoch for which the rank has executed step ``kind``."""
        v = 0
        for st in prog[:rank_pc]:
            if st[0] == kind:
                v = st[1]
        return v

    def inside(rank_pc: int, begin: str, end: str):
        """Epoch of an open begin/end section of the rank, or None."""
        open_e = None
        for st in prog[:rank_pc]:
            if st[0] == begin:
                open_e = st[1]
            elif st[0] == end:
                open_e = None
        return open_e

    while queue:
        pcs = queue.popleft()
        moved = False
        for r in range(W):
            if pcs[r] >= n:
                continue
            kind, e = prog[pcs[r]]
            peers = [p for p in range(W) if p != r]
            if kind == "wait_ready" and any(value(pcs[p], "ready") < e for p in peers):
                continue
            if kind == "wait_params" and any(value(pcs[p], "pushed") < e for p in peers):
                continue
            if kind == "wait_acks" and any(value(pcs[p], "ack") < e for p in peers):
                continue
            if kind == "reduce_begin":
                for p in peers:
                    # the peer's gradients of this step must be final: its backward of step e is over, and it has not
                    # started clearing or accumulating for a later step
                    if value(pcs[p], "fwd_end") < e:
                        raise Race(f"rank {r} reduces step {e} while rank {p} still accumulates it")
                    if value(pcs[p], "zero") >= e:
                        raise Race(f"rank {r} reduces step {e} after rank {p} cleared its gradients")
            if kind == "zero" or kind == "fwd_begin":
                for p in peers:
                    open_e = inside(pcs[p], "reduce_begin", "reduce_end")
                    if open_e is not None and (kind == "zero" or open_e < e):
                        raise Race(f"rank {r} {kind} step {e} while rank {p} reads its gradients of step {open_e}")
                    if kind == "zero" and value(pcs[p], "reduce_end") < e:
                        raise Race(f"rank {r} clears gradients of step {e} that rank {p} has not reduced yet")
            if kind == "fwd_begin" and e > 1:
                for p in peers:
                    if value(pcs[p], "push") < e - 1:
                        raise Race(f"rank {r} starts step {e} before rank {p}'s parameters of step {e - 1} arrived")
            if kind == "push":
                for p in peers:
                    open_e = inside(pcs[p], "fwd_begin", "fwd_end")
                    if open_e is not None and open_e <= e:
                        raise Race(f"rank {r} stores parameters of step {e} while rank {p} computes step {open_e} with them")
            moved = True
            nxt = pcs[:r] + (pcs[r] + 1,) + pcs[r + 1:]
            if nxt not in seen:
                seen.add(nxt)
                queue.append(nxt)
        if not moved and any(pc < n for pc in pcs):
            raise Stuck(str(pcs))
    return len(seen)


@pytest.mark.parametrize("W,steps", [(2, 3), (3, 2)])
def test_shard_collective_protocol_is_race_free(W, steps):
    assert explore(W, steps) > 10


def test_reduction_needs_the_ready_flags():
    with pytest.raises(Race):
        explore(2, 2, wait_ready=False)


def test_ready_flag_must_follow_the_backward():
    with pytest.raises(Race):
        explore(2, 2, ready_after_backward=False)


def test_clearing_gradients_needs_the_acknowledgements():
    # In the trainer's order (publish, wait for the peers' publications, then clear) the publication flags already
    # imply that every peer has finished reading; a caller that clears earlier depends on the acknowledgements.
    assert explore(2, 2, zero_before_push=True) > 10
    with pytest.raises(Race):
        explore(2, 2, zero_before_push=True, wait_acks=False)
    with pytest.raises(Race):
        explore(2, 2, wait_acks=False, wait_params=False)


def test_next_forward_needs_the_published_regions():
    with pytest.raises(Race):
        explore(2, 2, wait_params=False)
