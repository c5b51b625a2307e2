"""Exhaustive interleaving check of the flag protocol of the peer-memory exchanges (a stand-in for a race detector).

The model restates what the kernels of ``pithtrain_b200/csrc/ep_fused.cu`` do per use of a channel — two slots, one
epoch counter, per-(slot, source) ready flags in the receiver's memory, per-(slot, destination) acknowledgements in the
sender's memory:

    sender, epoch e, slot e % 2:   wait ack[slot][d] >= e - 2 for every d      (ep_wait_acks_kernel)
                                   store rows into d's partition [slot][me]    (ep_push_kernel / ep_return_kernel)
                                   release-store flag[slot][me] = e at d
    receiver, epoch e:             wait flag[slot][s] >= e for every s         (ep_wait_flags_kernel)
                                   read partitions [slot][*]                   (ep_compact_kernel / combine)
                                   release-store ack[slot][me] = e at every s  (ep_ack_kernel)

Every stream runs its steps in program order; a rank has one stream for both sides or one each; streams interleave
arbitrarily. The checker walks every reachable state and asserts: a partition is never written while its owner reads
it, a read sees exactly the epoch it waited for, and no state is stuck. The mutated protocols below (no acknowledgement wait, acknowledgement before the
read, one slot) must each be caught, which shows that the checker can see the races it is meant to exclude.
"""
from collections import deque
from typing import Dict, List, Optional, Tuple

import pytest


def program(rank: int, ep: int, epochs: int, *, wait_acks: bool = True, ack_after_read: bool = True, slots: int = 2,
            ack_lag: int = 2, streams: int = 1) -> List[List[Tuple]]:
    """The step lists of one rank: one list when sends and receives share a stream, two when the receive side runs on
    a stream of its own (so that the sender can run ahead of the local receiver)."""
    send: List[Tuple] = []
    recv: List[Tuple] = []
    both: List[Tuple] = []
    for e in range(1, epochs + 1):
        slot = e % slots
        s_steps: List[Tuple] = [("wait_ack", e, slot, ack_lag)] if wait_acks else []
        s_steps += [("write", e, slot, d) for d in range(ep)]
        s_steps.append(("flag_all", e, slot))
        r_steps: List[Tuple] = [("wait_flag", e, slot)]
        if not ack_after_read:
            r_steps.append(("ack_all", e, slot))
        r_steps += [("read_begin", e, slot), ("read_end", e, slot)]
        if ack_after_read:
            r_steps.append(("ack_all", e, slot))
        send += s_steps
        recv += r_steps
        both += s_steps + r_steps
    return [both] if streams == 1 else [send, recv]


class Violation(Exception):
    pass


def explore(ep: int, epochs: int, **mutation) -> int:
    """Breadth-first over all interleavings; returns the number of states. Raises ``Violation`` on a race, a stale
    read or a stuck state."""
    threads: List[Tuple[int, List[Tuple]]] = []  # (rank, steps)
    for r in range(ep):
        for steps in program(r, ep, epochs, **mutation):
            threads.append((r, steps))
    n = len(threads)

    def memory(pcs: Tuple[int, ...]):
        """Shared memory as a function of the program counters (each thread's stores are a prefix of its program)."""
        data: Dict[Tuple[int, int, int], int] = {}  # (owner, slot, src) -> epoch last written
        flag: Dict[Tuple[int, int, int], int] = {}  # (owner, slot, src) -> epoch
        ack: Dict[Tuple[int, int, int], int] = {}  # (owner = sender, slot, dst) -> epoch
        reading: Dict[Tuple[int, int], Optional[int]] = {}  # (owner, slot) -> epoch being read
        for (r, steps), pc in zip(threads, pcs):
            for st in steps[:pc]:
                kind = st[0]
                if kind == "write":
                    data[(st[3], st[2], r)] = st[1]
                elif kind == "flag_all":
                    for d in range(ep):
                        flag[(d, st[2], r)] = st[1]
                elif kind == "ack_all":
                    for s_ in range(ep):
                        ack[(s_, st[2], r)] = st[1]
                elif kind == "read_begin":
                    reading[(r, st[2])] = st[1]
                elif kind == "read_end":
                    reading[(r, st[2])] = None
        return data, flag, ack, reading

    start = tuple([0] * n)
    seen = {start}
    queue = deque([start])
    while queue:
        pcs = queue.popleft()
        data, flag, ack, reading = memory(pcs)
        moved = False
        for i, (r, steps) in enumerate(threads):
            if pcs[i] >= len(steps):
                continue
            st = steps[pcs[i]]
            kind, e, slot = st[0], st[1], st[2]
            if kind == "wait_ack":
                lag = st[3]
                if e > lag and any(ack.get((r, slot, d), 0) < e - lag for d in range(ep)):
                    continue  # blocked
            elif kind == "wait_flag":
                if any(flag.get((r, slot, s_), 0) < e for s_ in range(ep)):
                    continue
            elif kind == "write":
                d = st[3]
                if reading.get((d, slot)) is not None:
                    raise Violation(f"rank {r} writes epoch {e} into slot {slot} of rank {d} while {d} reads epoch {reading[(d, slot)]}")
                prev = data.get((d, slot, r), 0)
                if prev and ack.get((r, slot, d), 0) < prev:
                    raise Violation(f"rank {r} overwrites epoch {prev} in slot {slot} of rank {d} before it was consumed")
            elif kind == "read_begin":
                for s_ in range(ep):
                    if data.get((r, slot, s_), 0) != e:
                        raise Violation(f"rank {r} reads slot {slot} for epoch {e} but source {s_} holds epoch {data.get((r, slot, s_), 0)}")
            moved = True
            nxt = pcs[:i] + (pcs[i] + 1,) + pcs[i + 1:]
            if nxt not in seen:
                seen.add(nxt)
                queue.append(nxt)
        if not moved and any(pcs[i] < len(threads[i][1]) for i in range(n)):
            raise Violation(f"stuck at {pcs}")
    return len(seen)


@pytest.mark.parametrize("ep,epochs,streams", [(2, 6, 1), (3, 4, 1), (2, 4, 2)])
def test_two_slot_epoch_protocol_is_race_free(ep, epochs, streams):
    assert explore(ep, epochs, streams=streams) > 100


def test_one_stream_per_rank_synchronises_by_itself():
    """When every rank sends and receives each epoch in order on one stream, the exchange pattern alone keeps a sender
    two epochs behind every receiver: the acknowledgement wait never blocks. It is what makes the protocol safe when
    the two sides of a rank run on different streams (next test)."""
    assert explore(2, 5, wait_acks=False, streams=1) > 100


def test_without_the_acknowledgement_wait_a_sender_on_its_own_stream_overruns_the_reader():
    with pytest.raises(Violation, match="overwrites|while|holds"):
        explore(2, 4, wait_acks=False, streams=2)


def test_acknowledging_before_the_read_is_a_race():
    with pytest.raises(Violation, match="while|holds|overwrites"):
        explore(2, 4, ack_after_read=False, streams=2)


def test_one_slot_needs_the_acknowledgement_of_the_previous_epoch():
    # with a single slot, waiting for epoch e-2 lets a sender overwrite epoch e-1 that nobody has read yet ...
    with pytest.raises(Violation):
        explore(2, 4, slots=1, streams=2)
    # ... waiting for e-1 is correct again (and serialises sender and reader, which is why the kernels use two slots)
    assert explore(2, 4, slots=1, ack_lag=1, streams=2) > 10
