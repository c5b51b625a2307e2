"""Exhaustive interleaving check of the control words of the context-parallel payload exchange
(``parallel/cp_fused.py`` over ``csrc/symm.cu``): publish once, every peer pulls; gradient partials go back to the owner.

Per use (epoch ``e``, slot ``e & 1``) a rank runs on its stream, in program order:

    publish(e)          wait DONE[p] >= e - 2 for every p (this slot's previous payload has been read everywhere),
                        write the local payload into slot e & 1, release-store READY[me] = e on every rank
    pull / read(e, s)   for every other rank s: wait READY[s] >= e, read slot e & 1 of rank s
    finish(e)           release-store DONE[me] = e on every rank
    push_grad(e, o)     for every other rank o: wait GDONE[o] >= e - 2, write partition [e & 1][me] at rank o,
                        release-store GREADY[me] = e at rank o
    collect_grads(e)    wait GREADY[w] >= e for every writer w, read the partitions [e & 1][*], release-store
                        GDONE[me] = e on every rank

The forward of a use runs publish / pull / finish, its backward push_grad / collect_grads; a rank may be a whole use ahead
of a peer. The checker walks every reachable interleaving and asserts that a slot is never rewritten while a peer still
reads its previous content, that a read sees the epoch it waited for, and that partitions are not overwritten before the
owner has summed them. Removing a guard must be caught.
"""
from collections import deque
from typing import List, Tuple

import pytest


class Race(Exception):
    pass


class Stuck(Exception):
    pass


def program(cp: int, uses: int, *, wait_done: bool = True, wait_ready: bool = True, wait_gdone: bool = True,
            wait_gready: bool = True, slots: int = 2, payload: bool = True, grads: bool = True, pulls: bool = True) -> List[Tuple]:
    prog: List[Tuple] = []
    lag = slots  # a slot is reused every `slots` epochs
    for e in range(1, uses + 1):
        if payload:
            if wait_done and e > lag:
                prog.append(("wait_done", e - lag))
            prog += [("write", e), ("ready", e)]
            if pulls:
                if wait_ready:
                    prog.append(("wait_ready", e))
                prog += [("read_begin", e), ("read_end", e)]
            prog.append(("done", e))
        if grads:
            if wait_gdone and e > lag:
                prog.append(("wait_gdone", e - lag))
            prog += [("gwrite", e), ("gready", e)]
            if wait_gready:
                prog.append(("wait_gready", e))
            prog += [("gsum_begin", e), ("gsum_end", e), ("gdone", e)]
    return prog


def explore(cp: int, uses: int, **mut) -> int:
    slots = mut.get("slots", 2)
    idle = mut.pop("idle_rank", None)  # a rank that publishes but needs nobody's payload (every block of it masked out)
    progs = [program(cp, uses, pulls=(r != idle), **mut) for r in range(cp)]

    def value_of(r: int, pc: int, kind: str) -> int:
        v = 0
        for st in progs[r][:pc]:
            if st[0] == kind:
                v = st[1]
        return v

    start = tuple([0] * cp)
    seen = {start}
    queue = deque([start])
    while queue:
        pcs = queue.popleft()
        moved = False
        for r in range(cp):
            if pcs[r] >= len(progs[r]):
                continue
            kind, e = progs[r][pcs[r]]
            peers = [p for p in range(cp) if p != r]

            if kind == "wait_done" and any(value_of(p, pcs[p], "done") < e for p in peers):
                continue
            if kind == "wait_ready" and any(value_of(p, pcs[p], "ready") < e for p in peers):
                continue
            if kind == "wait_gdone" and any(value_of(p, pcs[p], "gdone") < e for p in peers):
                continue
            if kind == "wait_gready" and any(value_of(p, pcs[p], "gready") < e for p in peers):
                continue
            if kind == "write":
                for p in peers:
                    # peers that still read (or have yet to read) the payload this slot held `slots` epochs ago
                    old = e - slots
                    reads = any(st[0] == "read_end" for st in progs[p])
                    if old >= 1 and reads and value_of(p, pcs[p], "read_end") < old:
                        raise Race(f"rank {r} rewrites its slot for epoch {e} before rank {p} has read epoch {old}")
            if kind == "read_begin":
                for p in peers:
                    have = value_of(p, pcs[p], "write")
                    if have < e:
                        raise Race(f"rank {r} reads epoch {e} of rank {p}, which holds {have}")
                    if have >= e + slots:
                        raise Race(f"rank {r} reads epoch {e} of rank {p}, already overwritten by {have}")
            if kind == "gwrite":
                for p in peers:
                    old = e - slots
                    if old >= 1 and value_of(p, pcs[p], "gsum_end") < old:
                        raise Race(f"rank {r} rewrites its partition at rank {p} for epoch {e} before epoch {old} was summed")
            if kind == "gsum_begin":
                for p in peers:
                    have = value_of(p, pcs[p], "gwrite")
                    if have < e:
                        raise Race(f"rank {r} sums epoch {e} before rank {p} delivered it")
                    if have >= e + slots:
                        raise Race(f"rank {r} sums epoch {e}, partition of rank {p} already holds {have}")
            moved = True
            nxt = pcs[:r] + (pcs[r] + 1,) + pcs[r + 1:]
            if nxt not in seen:
                seen.add(nxt)
                queue.append(nxt)
        if not moved and any(pcs[i] < len(progs[i]) for i in range(cp)):
            raise Stuck(str(pcs))
    return len(seen)


@pytest.mark.parametrize("cp,uses", [(2, 5), (3, 3)])
def test_payload_and_gradient_routes_are_race_free(cp, uses):
    assert explore(cp, uses) > 10


def test_forward_only_use_is_race_free():
    # inference and the forward exchanges of a step: no gradient route keeps the ranks in step, only the DONE words do
    assert explore(2, 6, grads=False) > 10
    assert explore(3, 4, grads=False) > 10


def test_slot_reuse_needs_the_done_words():
    # When every rank pulls from every peer in every use, the READY handshakes alone keep two slots safe. A rank that
    # needs nobody's payload (all of its blocks masked out by a sliding window) has no such handshake and would run ahead:
    # the DONE words hold it back.
    assert explore(2, 4, grads=False, wait_done=False) > 10
    assert explore(2, 5, grads=False, idle_rank=0) > 10
    with pytest.raises(Race):
        explore(2, 5, grads=False, idle_rank=0, wait_done=False)


def test_pull_needs_the_ready_word():
    with pytest.raises(Race):
        explore(2, 2, wait_ready=False)


def test_partition_reuse_and_the_gdone_words():
    # Every rank is writer and owner in every use and an owner waits for all writers, so with two slots the GREADY
    # handshakes already order a rewrite behind the owner's sum; the GDONE wait is what makes a single slot safe.
    assert explore(2, 5, payload=False) > 10
    assert explore(2, 4, payload=False, wait_gdone=False) > 10
    assert explore(2, 4, payload=False, slots=1) > 10
    with pytest.raises(Race):
        explore(2, 4, payload=False, slots=1, wait_gdone=False)


def test_sum_needs_the_gready_words():
    with pytest.raises(Race):
        explore(2, 2, wait_gready=False)
