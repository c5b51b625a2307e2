"""Interleaving check of the mbarrier protocol of the attention forward kernel (``csrc/attention.cu``, two query tiles
per CTA), restated step by step with the kernel's barrier names, arrival counts and wait parities.

Agents: the producer warp, the two MMA-issuing threads (one per query tile, taking turns block by block), one in-order
"tensor pipe" per issuer that completes that thread's MMA batches and delivers its ``tcgen05.commit`` arrivals at some
later time, and one softmax agent per tile (the kernel's four warps arrive four times on a barrier of count 4; here one
agent and count 1). An mbarrier is modelled by its number of arrivals: phase ``p`` is complete after
``count * (p + 1)`` arrivals and ``wait(parity)`` passes when the phase in progress has the other parity, so a waiter
two phases behind is exposed as well. A commit covers every MMA its thread issued before it; a commit by a thread that
never issued an MMA does not arrive at all, which is why an issuer whose tile does not exist releases stages with a plain
arrive.

The checker walks every reachable interleaving and asserts that nobody is stuck and that buffers are used in order:
a K / V stage is refilled only after the MMAs of both tiles that read it completed, S is overwritten only after P of the
previous step was consumed, P halves are read only after they were written, O is rescaled only between P V batches.
Mutations of the protocol must be caught.
"""
from bisect import bisect_left
from collections import deque
from typing import Dict, List, Tuple

import pytest

KST = 2  # K / V ring depth of the (128, 128) configuration


class Stuck(Exception):
    pass


class Hazard(Exception):
    pass


def build(J: int, n0: int, n1: int, *, turns: bool = True, absent_tile_commits: bool = False, walk_ring_when_idle: bool = True,
          turn_parity_ok: bool = True, wait_second_half: bool = True):
    """Step lists for a CTA that walks ``J`` key tiles; tile ``t`` uses the first ``n_t`` of them (``n_t`` = 0: the tile
    does not exist, as for the odd last pair of a sequence)."""
    n = (n0, n1)
    agents: Dict[str, List[Tuple]] = {"prod": [], "iss0": [], "iss1": [], "pipe0": [], "pipe1": [], "soft0": [], "soft1": []}
    prod = agents["prod"]
    prod.append(("arrive", "q_full"))
    for c in range(J):
        s, ph = c % KST, (c // KST) & 1
        prod += [("wait", f"k_empty{s}", ph ^ 1), ("k_free", c), ("mark", f"K{c}"), ("arrive", f"k_full{s}"),
                 ("wait", f"v_empty{s}", ph ^ 1), ("v_free", c), ("mark", f"V{c}"), ("arrive", f"v_full{s}")]

    for t in (0, 1):
        iss, pipe = agents[f"iss{t}"], agents[f"pipe{t}"]
        exists = n[t] > 0
        seq = [0]

        def release(bar):
            # tcgen05.commit: arrives once this thread's MMAs so far are complete; without any MMA it never arrives
            if exists or absent_tile_commits:
                name = f"rel{t}_{seq[0]}"
                seq[0] += 1
                iss.append(("issue", name))
                pipe.append(("complete", name, [bar], exists))
            else:
                iss.append(("arrive", bar))

        def step_S(c):
            s = c % KST
            if c < n[t] or walk_ring_when_idle:
                iss.append(("wait", f"k_full{s}", (c // KST) & 1))
            if c < n[t]:
                iss.append(("need", f"K{c}"))
                if c > 0:
                    iss.append(("need", f"issued_PVb{t}_{c - 1}"))  # S overwrites P of the previous step: same thread, in order
                iss.append(("issue", f"S{t}_{c}"))
                pipe.append(("complete", f"S{t}_{c}", [f"s_full{t}"], True))
            release(f"k_empty{s}")

        iss.append(("wait", "q_full", 0))
        step_S(0)
        for c in range(J):
            s = c % KST
            if turns:
                if t == 1:
                    iss.append(("wait", "turn1", (c & 1) if turn_parity_ok else (c & 1) ^ 1))
                elif c > 0:
                    iss.append(("wait", "turn0", (c - 1) & 1))
            iss.append(("wait", f"v_full{s}", (c // KST) & 1))
            if c < n[t]:
                iss += [("wait", f"p_full{t}", c & 1), ("need", f"V{c}"), ("need", f"P1_{t}_{c}"), ("issue", f"PVa{t}_{c}")]
                pipe.append(("complete", f"PVa{t}_{c}", [], True))
                if wait_second_half:
                    iss.append(("wait", f"p_full2_{t}", c & 1))
                iss += [("need", f"P2_{t}_{c}"), ("issue", f"PVb{t}_{c}")]
                pipe.append(("complete", f"PVb{t}_{c}", [f"o_done{t}"] if c == n[t] - 1 else [], True))
            release(f"v_empty{s}")
            if c + 1 < J:
                step_S(c + 1)
            if turns:
                iss.append(("arrive", f"turn{1 - t}"))

        soft = agents[f"soft{t}"]
        for c in range(n[t]):
            soft += [("wait", f"s_full{t}", c & 1), ("need", f"done_S{t}_{c}")]
            if c > 0:
                # the rescale of O and the rewrite of P sit between the P V batches of steps c-1 and c
                soft.append(("need", f"done_PVb{t}_{c - 1}"))
            soft += [("forbid", f"issued_PVa{t}_{c}"), ("mark", f"P1_{t}_{c}"), ("arrive", f"p_full{t}"),
                     ("forbid", f"issued_PVb{t}_{c}"), ("mark", f"P2_{t}_{c}"), ("arrive", f"p_full2_{t}")]
        if n[t] > 0:
            soft += [("wait", f"o_done{t}", 0), ("need", f"done_PVb{t}_{n[t] - 1}"), ("mark", f"O_read{t}")]

    counts = {"q_full": 1, "turn0": 1, "turn1": 1}
    for s in range(KST):
        counts.update({f"k_full{s}": 1, f"v_full{s}": 1, f"k_empty{s}": 2, f"v_empty{s}": 2})  # both issuers release a stage
    for t in (0, 1):
        counts.update({f"s_full{t}": 1, f"p_full{t}": 1, f"p_full2_{t}": 1, f"o_done{t}": 1})
    return agents, counts, n


def explore(agents, counts, n) -> int:
    names = list(agents)
    steps = [agents[a] for a in names]
    # every fact has one producing step; a barrier's arrivals are the steps that name it
    fact_at: Dict[str, Tuple[int, int]] = {}
    arrive_at: Dict[str, List[List[int]]] = {b: [[] for _ in names] for b in counts}
    for ai, st_list in enumerate(steps):
        for i, st in enumerate(st_list):
            if st[0] == "mark":
                fact_at[st[1]] = (ai, i)
            elif st[0] == "issue":
                fact_at["issued_" + st[1]] = (ai, i)
            elif st[0] == "complete":
                fact_at["done_" + st[1]] = (ai, i)
                for b in st[2]:
                    arrive_at[b][ai].append(i)
            elif st[0] == "arrive":
                arrive_at[st[1]][ai].append(i)
    # a commit-only batch of a thread without MMAs never completes
    never = {st[1] for st_list in steps for st in st_list if st[0] == "complete" and not st[3]}

    def holds(fact, pcs):
        where = fact_at.get(fact)
        return where is not None and pcs[where[0]] > where[1]

    def arrivals(bar, pcs):
        return sum(bisect_left(idx, pcs[ai]) for ai, idx in enumerate(arrive_at[bar]))

    start = tuple([0] * len(names))
    seen = {start}
    queue = deque([start])
    while queue:
        pcs = queue.popleft()
        moved = False
        for i in range(len(names)):
            if pcs[i] >= len(steps[i]):
                continue
            st = steps[i][pcs[i]]
            kind = st[0]
            if kind == "wait":
                if ((arrivals(st[1], pcs) // counts[st[1]]) & 1) == st[2]:
                    continue
            elif kind == "complete":
                if st[1] in never or not holds("issued_" + st[1], pcs):
                    continue
            elif kind == "need":
                if not holds(st[1], pcs):
                    raise Hazard(f"{names[i]} needs {st[1]} at {dict(zip(names, pcs))}")
            elif kind == "forbid":
                if holds(st[1], pcs):
                    raise Hazard(f"{names[i]} runs after {st[1]} at {dict(zip(names, pcs))}")
            elif kind in ("k_free", "v_free"):
                prev = st[1] - KST
                for t in (0, 1):
                    if 0 <= prev < n[t]:
                        batch = f"done_S{t}_{prev}" if kind == "k_free" else f"done_PVb{t}_{prev}"
                        if not holds(batch, pcs):
                            raise Hazard(f"stage of key tile {prev} refilled for {st[1]} before {batch}")
            moved = True
            nxt = pcs[:i] + (pcs[i] + 1,) + pcs[i + 1:]
            if nxt not in seen:
                seen.add(nxt)
                queue.append(nxt)
        if not moved and any(pcs[i] < len(steps[i]) for i in range(len(names))):
            # pipes of commit-only batches that can never complete are allowed to stay behind only if nobody waits on them
            left = {names[i]: steps[i][pcs[i]] for i in range(len(names)) if pcs[i] < len(steps[i])}
            raise Stuck(f"no agent can move: {left}")
    return len(seen)


@pytest.mark.parametrize("J,n0,n1", [(1, 1, 1), (2, 1, 2), (3, 3, 3), (3, 2, 3), (4, 3, 4)])
def test_forward_protocol_has_no_deadlock_and_no_buffer_hazard(J, n0, n1):
    assert explore(*build(J, n0, n1)) > 10


@pytest.mark.parametrize("J,n0,n1", [(1, 1, 0), (3, 3, 0)])
def test_pair_with_an_absent_second_tile_completes(J, n0, n1):
    assert explore(*build(J, n0, n1)) > 10


def test_without_turns_the_protocol_is_still_safe():
    # the turns only order the two issuers for overlap; safety does not depend on them
    assert explore(*build(3, 2, 3, turns=False)) > 10


def test_issuer_of_an_absent_tile_must_not_release_by_commit():
    with pytest.raises(Stuck):  # its commits never arrive: the stages are never handed back to the producer
        explore(*build(3, 3, 0, absent_tile_commits=True))


def test_wrong_turn_parity_deadlocks():
    with pytest.raises(Stuck):
        explore(*build(2, 2, 2, turn_parity_ok=False))


def test_second_half_of_p_must_be_awaited():
    with pytest.raises(Hazard):  # the P V MMAs of keys 64..127 would read columns still holding scores
        explore(*build(2, 2, 2, wait_second_half=False))


def test_idle_issuer_must_follow_the_ring():
    # an issuer past its tile's last key tile still waits for every K stage. Without that wait (and without the turns,
    # which keep the issuers in step by themselves) it runs ahead, a stage's release counts two arrivals of the same
    # thread, and the producer refills a stage the other tile has not read yet.
    with pytest.raises((Hazard, Stuck)):
        explore(*build(5, 1, 5, walk_ring_when_idle=False, turns=False))
    assert explore(*build(5, 1, 5, walk_ring_when_idle=True, turns=False)) > 10


# ------------------------------------------------------------------------------------------------ backward
def build_bwd(N: int, *, wait_dk_done: bool = True, q_empty_count: int = 2, wait_dq_read: bool = True,
              wait_dp_read: bool = True, p_ready_slots: int = 2):
    """The barrier protocol of ``attn_bwd_kernel`` (``csrc/attention_bwd.cu``) for one key tile that meets ``N`` query
    tiles. Agents: producer, the "front" issuer (S^T, dP^T) and the "back" issuer (dV, dQ, dK) with one in-order pipe
    each, the compute warps (one agent; the kernel's eight warps arrive on barriers of count 8) and the dQ reduction
    warps (one agent for the kernel's four). TMEM regions R0 / R1 alternate: step n has S^T -> P^T -> dQ in R[n & 1] and
    dP^T in the other one, which S^T of step n+1 takes over."""
    ag: Dict[str, List[Tuple]] = {k: [] for k in ("prod", "front", "back", "pipeF", "pipeB", "comp", "red")}
    prod, front, back, comp, red = ag["prod"], ag["front"], ag["back"], ag["comp"], ag["red"]
    prod.append(("arrive", "kv_full"))
    for n in range(N):
        st = n & 1
        prod.append(("wait", f"q_empty{st}", ((n >> 1) & 1) ^ 1))
        if n >= 2:
            prod += [("need", f"done_S{n - 2}"), ("need", f"done_dK{n - 2}")]  # both readers of the Q stage finished
        prod += [("mark", f"Q{n}"), ("arrive", f"q_full{st}"), ("wait", "do_empty", (n & 1) ^ 1)]
        if n >= 1:
            prod += [("need", f"done_dP{n - 1}"), ("need", f"done_dV{n - 1}")]
        prod += [("mark", f"DO{n}"), ("arrive", "do_full")]

    def issue_S(n):
        front.append(("need", f"Q{n}"))
        if n >= 1:
            front.append(("need", f"dP_read{n - 1}"))  # S^T(n) takes the region dP^T(n-1) has left
        front.append(("issue", f"S{n}"))
        ag["pipeF"].append(("complete", f"S{n}", ["s_full", f"q_empty{n & 1}"], True))

    front += [("wait", "kv_full", 0), ("wait", "q_full0", 0)]
    issue_S(0)
    for n in range(N):
        front.append(("wait", "do_full", n & 1))
        if n > 0:
            if wait_dq_read:
                front.append(("wait", "dq_read", (n - 1) & 1))
            front.append(("need", f"dQ_read{n - 1}"))  # dP^T(n) takes the region dQ(n-1) was accumulated in
        front += [("need", f"DO{n}"), ("issue", f"dP{n}")]
        ag["pipeF"].append(("complete", f"dP{n}", ["dp_full", "do_empty"], True))
        if wait_dp_read:
            front.append(("wait", "dp_read", n & 1))
        if n + 1 < N:
            front.append(("wait", f"q_full{(n + 1) & 1}", ((n + 1) >> 1) & 1))
            issue_S(n + 1)

    back.append(("wait", "kv_full", 0))
    for n in range(N):
        pr, prp = (f"p_ready{n & 1}", (n >> 1) & 1) if p_ready_slots == 2 else ("p_ready0", n & 1)
        back += [("wait", "do_full", n & 1), ("wait", pr, prp), ("need", f"P{n}"), ("need", f"DO{n}"), ("issue", f"dV{n}")]
        ag["pipeB"].append(("complete", f"dV{n}", ["do_empty"], True))
        back += [("wait", f"q_full{n & 1}", (n >> 1) & 1), ("wait", "ds_ready", n & 1), ("need", f"dS{n}"), ("need", f"Q{n}"),
                 ("need", f"P_reread{n}"),  # dQ overwrites the region that still holds P^T: the compute warps have re-read it
                 ("issue", f"dQ{n}"), ("issue", f"dK{n}")]
        ag["pipeB"] += [("complete", f"dQ{n}", ["dq_full"], True), ("complete", f"dK{n}", ["dk_done", f"q_empty{n & 1}"], True)]
    back.append(("issue", "final"))
    ag["pipeB"].append(("complete", "final", ["all_done"], True))

    for n in range(N):
        comp += [("wait", "s_full", n & 1), ("wait", f"q_full{n & 1}", (n >> 1) & 1), ("need", f"done_S{n}"),
                 ("mark", f"P{n}"), ("arrive", f"p_ready{n & 1}" if p_ready_slots == 2 else "p_ready0"), ("wait", "dp_full", n & 1)]
        if n > 0 and wait_dk_done:
            comp.append(("wait", "dk_done", (n - 1) & 1))
        comp += [("need", f"done_dP{n}"), ("forbid", f"issued_dQ{n}"), ("mark", f"P_reread{n}"), ("mark", f"dP_read{n}"),
                 ("arrive", "dp_read")]
        if n > 0:
            comp += [("need", f"done_dQ{n - 1}"), ("need", f"done_dK{n - 1}")]  # both read the dS^T tile rewritten now
        comp += [("mark", f"dS{n}"), ("arrive", "ds_ready")]

    for n in range(N):
        red += [("wait", "dq_full", n & 1), ("need", f"done_dQ{n}"), ("forbid", f"issued_dP{n + 1}"), ("mark", f"dQ_read{n}"),
                ("arrive", "dq_read")]
    red += [("wait", "all_done", 0), ("need", f"done_dK{N - 1}"), ("need", f"done_dV{N - 1}")]

    counts = {b: 1 for b in ("kv_full", "q_full0", "q_full1", "do_full", "s_full", "dp_full", "p_ready0", "p_ready1", "dp_read", "ds_ready",
                             "dq_full", "dq_read", "all_done", "dk_done")}
    counts.update({"q_empty0": q_empty_count, "q_empty1": q_empty_count, "do_empty": 2})
    return ag, counts, (0, 0)


@pytest.mark.parametrize("N", [1, 2, 3, 4])
def test_backward_protocol_has_no_deadlock_and_no_buffer_hazard(N):
    assert explore(*build_bwd(N)) > 10


def test_backward_ds_tile_needs_the_dk_barrier():
    # dK is issued after dQ: the completion of dQ (which gates the next dP^T and through it the next dS^T) says nothing
    # about dK, which still reads the dS^T tile
    with pytest.raises(Hazard):
        explore(*build_bwd(3, wait_dk_done=False))


def test_backward_q_stage_needs_both_issuers():
    with pytest.raises((Hazard, Stuck)):
        explore(*build_bwd(4, q_empty_count=1))


def test_backward_dp_needs_the_dq_read_out():
    with pytest.raises(Hazard):
        explore(*build_bwd(3, wait_dq_read=False))


def test_backward_next_s_needs_the_dp_read_out():
    with pytest.raises(Hazard):
        explore(*build_bwd(3, wait_dp_read=False))


def test_backward_p_ready_needs_two_slots():
    # The compute warps do not depend on the back issuer between P^T of step n and P^T of step n+1 (S^T(n+1) and its
    # inputs come from the front issuer alone), so with a single barrier they could arrive for step n+1 before the back
    # issuer has looked at step n, which then waits on a phase parity that has already come round. Two barriers,
    # alternating by step, cannot alias: step n+2 needs dP^T(n+1), which needs dQ(n) read out, which needs the back issuer
    # past P^T(n).
    with pytest.raises(Stuck):
        explore(*build_bwd(2, p_ready_slots=1))
