"""Routing sort through the entry point that never allocates device memory.

Some embedders of the native library cannot call cudaMalloc when they need the sort (a stream
capture is open, or all device memory belongs to another allocator), so ``pt_route_sort_noalloc``
keeps its per-expert counters in a static device array inside the library. This test calls the
exported C symbol directly through ctypes, twice in a row with different inputs (the second call
sees whatever the first left in the shared scratch), and requires results identical to the
regular ``pt_route_sort`` entry point, whose scratch is a caller-provided tensor. It also checks
that a size beyond the static maximum is refused without touching the outputs.

The file name sorts last so that a run stopping at the first failure has already run every other
test; the test is self-contained and also passes alone in a fresh process.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu

MAX_EXPERTS = 1024  # PT_ROUTE_SORT_NOALLOC_MAX_EXPERTS


def _regular(L, eids, E, align, r_cap):
    n = eids.numel()
    dev = eids.device
    counts = torch.empty(E, dtype=torch.int32, device=dev)
    offs = torch.empty(E + 1, dtype=torch.int32, device=dev)
    ros = torch.empty(n, dtype=torch.int32, device=dev)
    sor = torch.empty(r_cap, dtype=torch.int32, device=dev)
    rc = L.pt_route_sort(eids.data_ptr(), None, n, E, align, counts.data_ptr(), counts.numel(), offs.data_ptr(), ros.data_ptr(),
                         sor.data_ptr(), r_cap, torch.cuda.current_stream().cuda_stream)
    assert rc == 0
    return offs, ros, sor


def _noalloc(L, eids, E, align, r_cap):
    n = eids.numel()
    dev = eids.device
    offs = torch.empty(E + 1, dtype=torch.int32, device=dev)
    ros = torch.empty(n, dtype=torch.int32, device=dev)
    sor = torch.empty(r_cap, dtype=torch.int32, device=dev)
    fn = L.pt_route_sort_noalloc
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p,
                   ctypes.c_void_p, ctypes.c_int, ctypes.c_void_p]
    rc = fn(eids.data_ptr(), n, E, align, offs.data_ptr(), ros.data_ptr(), sor.data_ptr(), r_cap,
            torch.cuda.current_stream().cuda_stream)
    return rc, offs, ros, sor


def test_route_sort_noalloc_matches_regular_entry_point():
    from pithtrain_b200 import _native

    L = _native.lib()
    torch.manual_seed(11)
    align = 16
    # two calls in a row; the second uses fewer experts and other data, so stale counters would show
    for n, k, E in [(4096, 8, 128), (777, 4, 32)]:
        eids = torch.randint(-1, E, (n * k,), device="cuda", dtype=torch.int32)
        r_cap = (n * k + align * E + 127) // 128 * 128
        ref_offs, ref_ros, ref_sor = _regular(L, eids, E, align, r_cap)
        rc, offs, ros, sor = _noalloc(L, eids, E, align, r_cap)
        assert rc == 0
        torch.cuda.synchronize()
        assert torch.equal(offs, ref_offs)
        assert torch.equal(ros, ref_ros)
        assert torch.equal(sor, ref_sor)


def test_route_sort_noalloc_rejects_oversize():
    from pithtrain_b200 import _native

    L = _native.lib()
    E = MAX_EXPERTS + 1
    eids = torch.zeros(64, device="cuda", dtype=torch.int32)
    r_cap = 64 + 16 * E
    rc, offs, ros, sor = _noalloc(L, eids, E, 16, r_cap)
    assert rc == -2


def test_route_sort_noalloc_accepts_the_maximum_expert_count():
    from pithtrain_b200 import _native

    L = _native.lib()
    torch.manual_seed(12)
    E, n, align = MAX_EXPERTS, 5000, 16
    eids = torch.randint(-1, E, (n,), device="cuda", dtype=torch.int32)
    r_cap = (n + align * E + 127) // 128 * 128
    ref_offs, ref_ros, ref_sor = _regular(L, eids, E, align, r_cap)
    rc, offs, ros, sor = _noalloc(L, eids, E, align, r_cap)
    assert rc == 0
    torch.cuda.synchronize()
    assert torch.equal(offs, ref_offs) and torch.equal(ros, ref_ros) and torch.equal(sor, ref_sor)


def test_route_sort_noalloc_writes_nothing_past_a_too_small_row_capacity():
    """Rows that do not fit: ``offs[E] > r_cap`` reports it and the words behind ``slot_of_row[r_cap]`` stay untouched."""
    from pithtrain_b200 import _native

    L = _native.lib()
    torch.manual_seed(13)
    E, n, align, r_cap, guard = 8, 1024, 16, 512, 256
    eids = torch.randint(0, E, (n,), device="cuda", dtype=torch.int32)
    offs = torch.empty(E + 1, dtype=torch.int32, device="cuda")
    ros = torch.empty(n, dtype=torch.int32, device="cuda")
    sor = torch.full((r_cap + guard,), 0x5A5A5A5A, dtype=torch.int32, device="cuda")
    fn = L.pt_route_sort_noalloc
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p,
                   ctypes.c_void_p, ctypes.c_int, ctypes.c_void_p]
    rc = fn(eids.data_ptr(), n, E, align, offs.data_ptr(), ros.data_ptr(), sor.data_ptr(), r_cap,
            torch.cuda.current_stream().cuda_stream)
    assert rc == 0
    torch.cuda.synchronize()
    assert int(offs[E]) > r_cap
    assert bool((sor[r_cap:] == 0x5A5A5A5A).all())
    _native.fetch_status()  # the regular path records the overflow in the status word; leave it clean for later tests
