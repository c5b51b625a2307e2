"""Property-based checks (hypothesis) of the index math and the numeric rules the kernels are tested against:
pipeline schedules, routing sort, expert-parallel send plans, the power-of-two scale rule, zigzag sharding."""
import math

import torch
from hypothesis import given, settings
from hypothesis import strategies as st

FAST = settings(max_examples=40, deadline=None)


@FAST
@given(P=st.integers(1, 8), extra=st.integers(0, 9))
def test_any_schedule_is_deadlock_free_and_balanced(P, extra):
    from pithtrain_b200.dualpipe.schedule import build_schedule, simulate

    N = 2 * P + extra
    simulate(P, N)  # raises on deadlock, unmatched messages or count mismatches
    for r in range(P):
        acts = build_schedule(P, r, N)
        kinds = [a.kind for a in acts]
        fwd = sum(k in ("F", "FB") for k in kinds)
        bwd = sum(k in ("B", "FB") for k in kinds)
        assert fwd == 2 * N and bwd == 2 * N
        deferred = sum(a.kind == "B" and a.zb for a in acts)
        assert deferred == kinds.count("W")  # every deferred weight-gradient chunk is drained by exactly one W


@FAST
@given(n=st.integers(1, 70), k=st.integers(1, 6), E=st.integers(1, 24), seed=st.integers(0, 10 ** 6), drop=st.floats(0, 0.5))
def test_route_sort_invariants(n, k, E, seed, drop):
    from pithtrain_b200.ops.moe import ALIGN, route_sort, sorted_capacity

    g = torch.Generator().manual_seed(seed)
    eids = torch.randint(0, E, (n, k), generator=g, dtype=torch.int32)
    eids[torch.rand(n, k, generator=g) < drop] = -1
    offs, row_of_slot, slot_of_row = route_sort(eids, E)
    flat = eids.flatten()
    assert int(offs[0]) == 0 and slot_of_row.numel() == sorted_capacity(n * k, E) and int(offs[-1]) <= slot_of_row.numel()
    for e in range(E):
        a, b = int(offs[e]), int(offs[e + 1])
        assert (b - a) % ALIGN == 0 and b - a >= int((flat == e).sum())
        live = slot_of_row[a:b][slot_of_row[a:b] >= 0]
        assert torch.equal(flat[live.long()], torch.full_like(live, e))
        assert torch.equal(live, live.sort().values) and live.numel() == int((flat == e).sum())
    valid = flat >= 0
    assert bool((row_of_slot[~valid] == -1).all())
    assert torch.equal(slot_of_row[row_of_slot[valid].long()].long(), torch.nonzero(valid).flatten())
    assert int((slot_of_row >= 0).sum()) == int(valid.sum())


@FAST
@given(m=st.integers(0, 60), k=st.integers(1, 6), per=st.integers(1, 6), ep=st.integers(1, 6), seed=st.integers(0, 10 ** 6))
def test_send_plan_invariants(m, k, per, ep, seed):
    from pithtrain_b200.parallel.ep import build_send_side

    E = per * ep
    k = min(k, E)
    g = torch.Generator().manual_seed(seed)
    idx = (torch.stack([torch.randperm(E, generator=g)[:k] for _ in range(m)]) if m else torch.zeros(0, k, dtype=torch.int64)).int()
    tok, pos, eids, counts = build_send_side(idx, E, ep)
    dest = idx.long() // per
    assert counts.tolist() == [int((dest == r).any(1).sum()) if m else 0 for r in range(ep)]
    assert tok.numel() == int(counts.sum()) == eids.shape[0]
    assert int((eids >= 0).sum()) == m * k and int(eids.max().item() if eids.numel() else -1) < per
    # rows are grouped by destination, tokens ascending inside a destination
    bounds = torch.cumsum(counts, 0).tolist()
    lo = 0
    for r, hi in enumerate(bounds):
        t = tok[lo:hi].long()
        assert torch.equal(t, t.sort().values) and len(set(t.tolist())) == t.numel()
        assert bool(((dest[t] == r).any(1)).all()) if t.numel() else True
        lo = hi
    assert torch.equal((pos >= 0), (dest.unsqueeze(-1) == torch.arange(ep)).any(1)) if m else pos.numel() == 0


@FAST
@given(x=st.floats(min_value=1e-12, max_value=3e38, allow_nan=False, allow_infinity=False))
def test_pow2_scale_is_the_smallest_power_of_two_that_fits(x):
    from pithtrain_b200.ops.quant import pow2_scale_ref

    amax = torch.tensor([x], dtype=torch.float32)
    s = float(pow2_scale_ref(amax))
    a = max(float(amax), 1e-4)
    exp = math.log2(s)
    assert exp == round(exp)
    target = float(torch.tensor(a, dtype=torch.float32) * torch.tensor(1.0 / 448.0, dtype=torch.float32))
    if s < 2.0 ** 126:  # below the clamp at the top of the exponent range
        assert s >= target and s / 2 < target  # ceil to a power of two; exact powers stay
    assert a / s <= 448.0 * (1 + 2 ** -20) or s >= 2.0 ** 126


@FAST
@given(cp=st.integers(1, 8), blocks=st.integers(1, 5))
def test_zigzag_blocks_partition_the_sequence_and_balance_causal_work(cp, blocks):
    """Rank r holds blocks r and 2cp-1-r: a partition of the sequence with the same causal work (sum of key counts)
    on every rank."""
    S = 2 * cp * blocks * 4
    b = S // (2 * cp)
    owned = [list(range(r * b, (r + 1) * b)) + list(range((2 * cp - 1 - r) * b, (2 * cp - r) * b)) for r in range(cp)]
    flat = sorted(p for o in owned for p in o)
    assert flat == list(range(S))
    work = [sum(p + 1 for p in o) for o in owned]
    assert max(work) - min(work) == 0


@FAST
@given(m_tiles=st.integers(1, 40), n_tiles=st.integers(1, 40))
def test_supergrouped_tile_order_visits_every_tile_once(m_tiles, n_tiles):
    """The dense tile order of ``csrc/gemm.cu`` / ``csrc/gemm_2cta.cu`` (row tiles in supergroups of eight, so that CTAs
    running together share A rows and B columns in L2), restated: linear index -> (row tile, column tile) is a
    bijection."""
    GROUP = 8
    seen = set()
    for t in range(m_tiles * n_tiles):
        per = GROUP * n_tiles
        gid = t // per
        first_m = gid * GROUP
        gsz = min(m_tiles - first_m, GROUP)
        local = t - gid * per
        mt, nt = first_m + local % gsz, local // gsz
        assert 0 <= mt < m_tiles and 0 <= nt < n_tiles
        seen.add((mt, nt))
    assert len(seen) == m_tiles * n_tiles
