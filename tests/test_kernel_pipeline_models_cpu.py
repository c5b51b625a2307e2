"""Interleaving check of the mbarrier protocol of ``csrc/gemm_2cta.cu`` (two CTAs: producers, leader MMA thread, tensor
pipe, epilogues), restated step by step with the kernel's barrier names, arrival counts and wait parities. (The
attention forward kernel has its own model in ``tests/test_attention_pipeline_model_cpu.py``.)

An mbarrier is modelled by its arrival count: phase ``p`` has completed once ``count * (p + 1)`` arrivals happened, and
``wait(parity)`` passes when the current (incomplete) phase has the other parity, which is also what makes a waiter
that falls two phases behind see the wrong phase, so the model exposes that mistake too. ``tcgen05.commit`` arrivals are
asynchronous: they happen when a separate "tensor pipe" agent completes the batch, any time after it was issued.
The checker walks every reachable interleaving and asserts that no agent is stuck and that every buffer is used in
order. Mutations (a missing commit to the peer, a wrong arrival count) must be caught.
"""
from collections import deque
from typing import Dict, List, Tuple

import pytest

class Stuck(Exception):
    pass


class Hazard(Exception):
    pass


def explore_agents(agents, counts, issuer: str = "mma") -> int:
    """Walk every interleaving of the agents' step lists. Step kinds: ``wait`` (barrier, parity), ``arrive`` (barrier),
    ``issue`` (batch) by the ``issuer``, ``complete`` (batch, barriers) by a pipe agent once the batch was issued,
    ``mark`` (fact), ``need`` / ``forbid`` (fact)."""
    names = list(agents)
    steps = [agents[n] for n in names]
    issue_index = {st[1]: i for i, st in enumerate(agents[issuer]) if st[0] == "issue"}

    def facts(pcs):
        arrivals: Dict[str, int] = {}
        marks = set()
        for a, pc in zip(names, pcs):
            for st in agents[a][:pc]:
                if st[0] == "arrive":
                    arrivals[st[1]] = arrivals.get(st[1], 0) + 1
                elif st[0] == "mark":
                    marks.add(st[1])
                elif st[0] == "issue":
                    marks.add("issued_" + st[1])
                elif st[0] == "complete":
                    marks.add("done_" + st[1])
                    for b in st[2]:
                        arrivals[b] = arrivals.get(b, 0) + 1
        return arrivals, marks

    start = tuple([0] * len(names))
    seen = {start}
    queue = deque([start])
    while queue:
        pcs = queue.popleft()
        arrivals, marks = facts(pcs)
        moved = False
        for i, a in enumerate(names):
            if pcs[i] >= len(steps[i]):
                continue
            st = steps[i][pcs[i]]
            kind = st[0]
            if kind == "wait":
                phase_bit = (arrivals.get(st[1], 0) // counts[st[1]]) & 1
                if phase_bit == st[2]:
                    continue  # the phase with this parity has not completed
            elif kind == "complete":
                if pcs[names.index(issuer)] <= issue_index[st[1]]:
                    continue  # not issued yet
            elif kind == "need":
                if st[1] not in marks:
                    raise Hazard(f"{a} needs {st[1]} at {pcs}")
            elif kind == "forbid":
                if st[1] in marks:
                    raise Hazard(f"{a} runs while {st[1]} at {pcs}")
            moved = True
            nxt = pcs[:i] + (pcs[i] + 1,) + pcs[i + 1:]
            if nxt not in seen:
                seen.add(nxt)
                queue.append(nxt)
        if not moved and any(pcs[i] < len(steps[i]) for i in range(len(names))):
            raise Stuck(f"no agent can move at {dict(zip(names, pcs))}")
    return len(seen)


# ------------------------------------------------------------------------------------------------ 2-CTA GEMM
def build_gemm_pair(tiles: int, num_kb: int, stages: int, *, peer_commit: bool = True, tmem_empty_count: int = 2):
    """The barrier protocol of ``csrc/gemm_2cta.cu`` for one CTA pair. Barriers named ``x@r`` live in CTA ``r``.
    ``full[s]@0`` completes on the leader producer's arrival plus the transaction bytes of both CTAs (the peer's bytes
    are modelled as a second arrival), ``empty[s]@r`` and ``tmem_full[b]@r`` receive one commit each from the leader's MMA thread,
    ``tmem_empty[b]@0`` receives one arrival per epilogue group of the pair (the kernel counts 8 warps; 2 groups here)."""
    agents = {"prod0": [], "prod1": [], "mma": [], "pipe": [], "epi0": [], "epi1": []}
    counts = {}
    for s in range(stages):
        counts[f"full{s}@0"] = 2  # the leader's arrival and, standing in for the peer's transaction bytes, one from CTA 1
        counts[f"empty{s}@0"] = counts[f"empty{s}@1"] = 1
    for b in range(2):
        counts[f"tmem_full{b}@0"] = counts[f"tmem_full{b}@1"] = 1
        counts[f"tmem_empty{b}@0"] = tmem_empty_count
    it = 0
    for t in range(tiles):
        acc = t & 1
        agents["mma"] += [("wait", f"tmem_empty{acc}@0", ((t >> 1) & 1) ^ 1)]
        if t >= 2:
            agents["mma"] += [("need", f"acc_read{t - 2}@0"), ("need", f"acc_read{t - 2}@1")]
        for kb in range(num_kb):
            s, ph = it % stages, (it // stages) & 1
            for r in (0, 1):
                steps = [("wait", f"empty{s}@{r}", ph ^ 1)]
                if it >= stages:
                    steps.append(("need", f"done_mma{it - stages}"))  # the stage's previous contents were consumed
                steps += [("mark", f"loaded{it}@{r}"), ("arrive", f"full{s}@0")]
                agents[f"prod{r}"] += steps
            agents["mma"] += [("wait", f"full{s}@0", ph), ("need", f"loaded{it}@0"), ("need", f"loaded{it}@1"), ("issue", f"mma{it}")]
            arrives = [f"empty{s}@0"] + ([f"empty{s}@1"] if peer_commit else [])
            agents["pipe"].append(("complete", f"mma{it}", arrives))
            it += 1
        agents["mma"].append(("issue", f"tile{t}"))
        agents["pipe"].append(("complete", f"tile{t}", [f"tmem_full{acc}@0"] + ([f"tmem_full{acc}@1"] if peer_commit else [])))
        for r in (0, 1):
            agents[f"epi{r}"] += [("wait", f"tmem_full{acc}@{r}", (t >> 1) & 1), ("need", f"done_tile{t}"),
                                  ("mark", f"acc_read{t}@{r}"), ("arrive", f"tmem_empty{acc}@0")]
    return agents, counts


@pytest.mark.parametrize("tiles,num_kb,stages", [(1, 3, 2), (3, 2, 2), (4, 3, 5), (5, 1, 3)])
def test_two_cta_gemm_protocol_has_no_deadlock_and_no_hazard(tiles, num_kb, stages):
    agents, counts = build_gemm_pair(tiles, num_kb, stages)
    assert explore_agents(agents, counts) > 10


def test_two_cta_gemm_needs_the_commit_to_the_peer():
    agents, counts = build_gemm_pair(2, 3, 2, peer_commit=False)
    with pytest.raises(Stuck):  # CTA 1 never sees its stages released or its accumulator ready
        explore_agents(agents, counts)


def test_two_cta_gemm_accumulator_needs_both_epilogues():
    agents, counts = build_gemm_pair(4, 1, 2, tmem_empty_count=1)
    with pytest.raises((Hazard, Stuck)):  # one arrival per phase lets the MMA overwrite rows the other CTA still reads
        explore_agents(agents, counts)
