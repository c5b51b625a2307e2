"""DualPipeV schedule as data.

``build_schedule(pp_size, pp_rank, num_chunks)`` returns the rank's list of :class:`Action` — the
eight-phase bidirectional V schedule with zero-bubble weight phases (phases and counts as in
pithtrain/dualpipe/dualpipev.py:544-610 of the reference, which follows DeepSeek's DualPipeV). Keeping
the schedule as a pure function makes it checkable without GPUs: :func:`simulate` replays all ranks'
action lists against each other with blocking message semantics and reports deadlocks, unmatched
messages and ordering violations.

Phases are 0 (first local chunk, stage ``rank``) and 1 (second local chunk, stage ``2P-1-rank``).
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Tuple


@dataclass(frozen=True)
class Action:
    kind: str  # "F", "B", "W", "FB", "SEND_F", "SEND_B", "RECV_F"
    phase: int = 0  # F/B/SEND/RECV phase; for FB the forward phase
    bphase: int = 0  # FB only: backward phase
    recv: bool = True  # F: post recv of the input; B: post recv of the output grad; FB: recv of the forward input
    send: bool = True  # F: post send of the output; B: post send of the input grad
    zb: bool = False  # B: defer weight gradients to a later W action

    def __repr__(self) -> str:  # compact, for test failure messages
        if self.kind == "FB":
            return f"FB({self.phase},{self.bphase}{'' if self.recv else ',norecv'})"
        if self.kind == "W":
            return "W"
        flags = "".join([("" if self.recv else "-r"), ("" if self.send else "-s"), ("z" if self.zb else "")])
        return f"{self.kind}{self.phase}{flags}"


def build_schedule(pp_size: int, pp_rank: int, num_chunks: int) -> List[Action]:
    P, R, N = pp_size, pp_rank, num_chunks
    assert N >= 2 * P, f"num_chunks ({N}) must be at least 2 * pp_size ({2 * P})"
    last = R == P - 1
    acts: List[Action] = []
    # 1: nF0
    for _ in range(2 * (P - R - 1)):
        acts.append(Action("F", 0))
    # 2: nF0F1
    n2 = R + 1
    acts.append(Action("RECV_F", 0))
    for i in range(n2):
        acts.append(Action("F", 0, recv=False, send=False))
        acts.append(Action("RECV_F", 0))  # the last one is consumed by the first steady-state forward
        acts.append(Action("F", 1, send=(not last) or (i < n2 - 1)))
        acts.append(Action("SEND_F", 0))
    # 3: nB1W1F1
    for _ in range(P - R - 1):
        acts.append(Action("B", 1, zb=True))
        acts.append(Action("RECV_F", 1))
        acts.append(Action("W"))
        acts.append(Action("F", 1, recv=False))
    # 4: nF0B1F1B0 (steady state)
    n4 = N - 2 * P + R + 1
    for i in range(n4):
        if i == 0:
            if last:
                # the rank that turns phase 0 into phase 1 cannot overlap its first pair
                acts.append(Action("F", 0, recv=False, send=False))
                acts.append(Action("SEND_F", 1))
                acts.append(Action("B", 1, send=False))
                acts.append(Action("SEND_F", 0))
                acts.append(Action("SEND_B", 1))
            else:
                acts.append(Action("FB", 0, 1, recv=False))
        else:
            acts.append(Action("FB", 0, 1))
        acts.append(Action("FB", 1, 0))
    # 5: nB1F1B0
    for _ in range(P - R - 1):
        acts.append(Action("B", 1))
        acts.append(Action("FB", 1, 0))
    # 6: nB1B0, second half with deferred weight gradients
    n6 = R + 1
    zb = False
    for i in range(n6):
        if i == n6 // 2 and R % 2 == 1:
            zb = True
        acts.append(Action("B", 1, zb=zb))
        if i == n6 // 2 and R % 2 == 0:
            zb = True
        acts.append(Action("B", 0, zb=zb))
    # 7: nWB0
    for _ in range(P - R - 1):
        acts.append(Action("W"))
        acts.append(Action("B", 0, zb=True))
    # 8: nW
    for _ in range(R + 1):
        acts.append(Action("W"))
    return [a for a in acts if a.kind != "NOP"]


# ------------------------------------------------------------------------------------------------
# Message model shared by the executor and the simulator
# ------------------------------------------------------------------------------------------------
def forward_src(P: int, R: int, phase: int):
    """Rank the forward input of ``phase`` comes from, or None (data loader / local hand-over)."""
    if (R == 0 and phase == 0) or (R == P - 1 and phase == 1):
        return None
    return R - 1 if phase == 0 else R + 1


def forward_dst(P: int, R: int, phase: int):
    if (R == 0 and phase == 1) or (R == P - 1 and phase == 0):
        return None
    return R + 1 if phase == 0 else R - 1


def backward_src(P: int, R: int, phase: int):
    """Rank the output gradient of ``phase`` comes from (= where the forward output went)."""
    return forward_dst(P, R, phase)


def backward_dst(P: int, R: int, phase: int):
    return forward_src(P, R, phase)


def simulate(pp_size: int, num_chunks: int) -> Dict[str, int]:
    """Replay every rank's schedule with the executor's communication protocol.

    Sends and receives are posted in program order and committed in batches exactly as the executor
    does (all ops pending at the start of a compute action are committed together and waited for).
    A batch completes when every receive in it has a matching send posted by the peer. Raises
    ``RuntimeError`` on deadlock or on any count mismatch; returns per-rank statistics.
    """
    P, N = pp_size, num_chunks
    scheds = [build_schedule(P, r, N) for r in range(P)]
    pc = [0] * P
    # message queues: (src, dst, tag) -> number of sends committed
    sent: Dict[Tuple[int, int, str], int] = {}
    recvd: Dict[Tuple[int, int, str], int] = {}
    pending_ops: List[List[Tuple[str, int, str]]] = [[] for _ in range(P)]  # (op, peer, tag)
    waiting: List[List[Tuple[int, str]]] = [[] for _ in range(P)]  # receives of the batch in flight
    f_done = [[0, 0] for _ in range(P)]
    b_done = [[0, 0] for _ in range(P)]
    w_queue = [0] * P
    w_done = [0] * P

    def post_recv_f(r, ph):
        s = forward_src(P, r, ph)
        if s is not None:
            pending_ops[r].append(("recv", s, f"F{ph}"))

    def post_send_f(r, ph):
        d = forward_dst(P, r, ph)
        if d is not None:
            pending_ops[r].append(("send", d, f"F{ph}"))

    def post_recv_b(r, ph):
        s = backward_src(P, r, ph)
        if s is not None:
            pending_ops[r].append(("recv", s, f"B{ph}"))

    def post_send_b(r, ph):
        d = backward_dst(P, r, ph)
        if d is not None:
            pending_ops[r].append(("send", d, f"B{ph}"))

    def commit(r):
        for op, peer, tag in pending_ops[r]:
            if op == "send":
                sent[(r, peer, tag)] = sent.get((r, peer, tag), 0) + 1
            else:
                waiting[r].append((peer, tag))
        pending_ops[r] = []

    def batch_ready(r):
        need: Dict[Tuple[int, int, str], int] = {}
        for peer, tag in waiting[r]:
            key = (peer, r, tag)
            need[key] = need.get(key, 0) + 1
        return all(sent.get(k, 0) - recvd.get(k, 0) >= n for k, n in need.items())

    def consume(r):
        for peer, tag in waiting[r]:
            key = (peer, r, tag)
            recvd[key] = recvd.get(key, 0) + 1
        waiting[r] = []

    state = ["issue"] * P  # "issue": next action not started; "wait": batch committed, waiting
    progress = True
    while progress:
        progress = False
        for r in range(P):
            while pc[r] < len(scheds[r]):
                a = scheds[r][pc[r]]
                if state[r] == "issue":
                    if a.kind == "RECV_F":
                        post_recv_f(r, a.phase); pc[r] += 1; progress = True; continue
                    if a.kind == "SEND_F":
                        post_send_f(r, a.phase); pc[r] += 1; progress = True; continue
                    if a.kind == "SEND_B":
                        post_send_b(r, a.phase); pc[r] += 1; progress = True; continue
                    if a.kind == "F" and a.recv:
                        post_recv_f(r, a.phase)
                    if a.kind == "B" and a.recv:
                        post_recv_b(r, a.phase)
                    if a.kind == "FB":
                        if a.recv:
                            post_recv_f(r, a.phase)
                        post_recv_b(r, a.bphase)
                    commit(r)
                    state[r] = "wait"
                if not batch_ready(r):
                    break
                consume(r)
                # compute
                if a.kind in ("F", "FB"):
                    f_done[r][a.phase] += 1
                if a.kind == "B" or a.kind == "FB":
                    ph = a.phase if a.kind == "B" else a.bphase
                    if b_done[r][ph] >= f_done[r][ph]:
                        raise RuntimeError(f"rank {r}: backward of phase {ph} before its forward ({a})")
                    b_done[r][ph] += 1
                    if a.kind == "B" and a.zb:
                        w_queue[r] += 1
                if a.kind == "W":
                    if w_queue[r] <= w_done[r]:
                        raise RuntimeError(f"rank {r}: W with an empty weight-gradient queue")
                    w_done[r] += 1
                # sends after compute
                if a.kind == "F" and a.send:
                    post_send_f(r, a.phase)
                if a.kind == "B" and a.send:
                    post_send_b(r, a.phase)
                if a.kind == "FB":
                    post_send_f(r, a.phase)
                    post_send_b(r, a.bphase)
                pc[r] += 1
                state[r] = "issue"
                progress = True
    for r in range(P):
        if pc[r] < len(scheds[r]):
            raise RuntimeError(f"deadlock: rank {r} stuck at action {pc[r]} {scheds[r][pc[r]]} of {len(scheds[r])}")
        if pending_ops[r]:
            # trailing sends are flushed by the executor's final commit
            commit(r)
    for r in range(P):
        for ph in (0, 1):
            if f_done[r][ph] != N or b_done[r][ph] != N:
                raise RuntimeError(f"rank {r} phase {ph}: {f_done[r][ph]} forwards / {b_done[r][ph]} backwards, expected {N}")
        if w_queue[r] != w_done[r]:
            raise RuntimeError(f"rank {r}: {w_queue[r]} deferred weight chunks but {w_done[r]} W actions")
    for key, n in sent.items():
        if recvd.get(key, 0) != n:
            raise RuntimeError(f"unmatched messages on {key}: sent {n}, received {recvd.get(key, 0)}")
    return {"actions": sum(len(s) for s in scheds), "messages": sum(sent.values())}
