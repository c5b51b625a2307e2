"""Context-parallel payload exchange over peer memory: publish once, every peer pulls directly.

The NCCL ring forwards K/V (or the MLA latent) hop by hop, so step ``i`` of ring attention cannot
start before ``i`` sequential transfers finished. Here every rank copies its payload into a symmetric
buffer once and flags it; a peer that needs the block of rank ``src`` waits for that one flag and
reads the block straight from ``src``'s memory over NVLink (a copy kernel on a side stream, so the
pull of step ``i+1`` overlaps the attention of step ``i``). Gradients take the reverse route: the
partial dK/dV computed against ``src``'s block is stored into a per-writer partition at the owner,
which sums the partitions in rank order (deterministic) once all writers have flagged.

Control words (``unsigned``, one block per rank, system-scope release/acquire):
``READY[r]`` epoch whose payload rank ``r`` published · ``DONE[r]`` epoch whose payload rank ``r``
finished reading everywhere · ``GREADY[w]`` epoch whose gradient partial writer ``w`` delivered to
this rank · ``GDONE[o]`` epoch whose partials owner ``o`` has consumed. Two slots per buffer; slot
``epoch & 1`` is reused only after the matching DONE/GDONE words reached ``epoch - 2``. Every wait is
a bounded in-kernel spin that reports through the library's status word.

Replaces the ``batch_isend_irecv`` rotation of the reference (pithtrain/operators/ring_attention.py:79-104,
275-277, 671-697).
"""

from __future__ import annotations

import ctypes
from typing import Dict, List, Sequence, Tuple

import torch
import torch.distributed as dist

from .. import _native
from .symm_mem import SymmetricBuffer

READY, DONE, GREADY, GDONE, CTL_WORDS = 0, 32, 64, 96, 128


def _align(n: int, a: int = 256) -> int:
    return (n + a - 1) // a * a


class PayloadExchange:
    def __init__(self, group, cp: int, rank: int, shapes: Sequence[Tuple[int, ...]], dtypes: Sequence[torch.dtype],
                 device, with_grads: bool) -> None:
        assert cp <= 32
        self.group, self.cp, self.rank, self.device = group, cp, rank, device
        self.shapes, self.dtypes = [tuple(s) for s in shapes], list(dtypes)
        self.offsets, off = [], 0
        for s, dt in zip(self.shapes, self.dtypes):
            self.offsets.append(off)
            n = 1
            for x in s:
                n *= x
            off = _align(off + n * torch.empty((), dtype=dt).element_size())
        self.slot_bytes = off
        self.buf = SymmetricBuffer(2 * self.slot_bytes, group, device, "context-parallel payload")
        self.ctl = SymmetricBuffer(CTL_WORDS * 4, group, device, "context-parallel control")
        self._ctl_ptrs = (ctypes.c_void_p * cp)(*self.ctl.peer_ptrs)
        self.with_grads = with_grads
        if with_grads:
            self.g_offsets, off = [], 0
            for s in self.shapes:
                self.g_offsets.append(off)
                n = 1
                for x in s:
                    n *= x
                off = _align(off + n * 4)
            self.g_part_bytes = off
            self.gbuf = SymmetricBuffer(2 * cp * self.g_part_bytes, group, device, "context-parallel gradients")
        self.epoch = 0
        self.side = torch.cuda.Stream(device=device)

    # ------------------------------------------------------------------ helpers
    def _signal(self, ptrs, n: int, index: int, value: int, stream) -> None:
        _native.check(_native.lib().pt_symm_signal(ctypes.addressof(ptrs), n, index, value, stream), "pt_symm_signal")

    def _wait(self, index: int, count: int, value: int, stream) -> None:
        _native.check(_native.lib().pt_symm_wait(self.ctl.local_ptr, index, count, value, stream), "pt_symm_wait")

    def _copy(self, dst_ptr: int, src_ptr: int, nbytes: int, stream, max_ctas: int = 0) -> None:
        assert nbytes % 16 == 0, "payload tensors must be multiples of 16 bytes"
        _native.check(_native.lib().pt_symm_copy(dst_ptr, src_ptr, nbytes, max_ctas, stream), "pt_symm_copy")

    def _nbytes(self, j: int) -> int:
        n = 1
        for x in self.shapes[j]:
            n *= x
        return n * torch.empty((), dtype=self.dtypes[j]).element_size()

    # ------------------------------------------------------------------ payload
    def publish(self, tensors: Sequence[torch.Tensor]) -> int:
        """Copy the local payload into this epoch's slot and flag it on every rank."""
        st = _native.stream_ptr()
        self.epoch += 1
        e = self.epoch
        if e > 2:
            self._wait(DONE, self.cp, e - 2, st)  # everybody finished reading this slot's previous content
        base = self.buf.local_ptr + (e & 1) * self.slot_bytes
        for j, t in enumerate(tensors):
            t = t.contiguous()
            assert tuple(t.shape) == self.shapes[j] and t.dtype == self.dtypes[j]
            assert t.data_ptr() % 16 == 0
            self._copy(base + self.offsets[j], t.data_ptr(), self._nbytes(j), st)
        self._signal(self._ctl_ptrs, self.cp, READY + self.rank, e, st)
        return e

    def pull(self, src: int, epoch: int) -> Tuple[List[torch.Tensor], torch.cuda.Event]:
        """Fetch the payload of ``src`` on the side stream; pair with :meth:`wait_pull` before use."""
        out = [torch.empty(s, dtype=dt, device=self.device) for s, dt in zip(self.shapes, self.dtypes)]
        self.side.wait_stream(torch.cuda.current_stream(self.device))
        with torch.cuda.stream(self.side):
            st = self.side.cuda_stream
            self._wait(READY + src, 1, epoch, st)
            base = self.buf.peer_ptrs[src] + (epoch & 1) * self.slot_bytes
            for j, t in enumerate(out):
                # a bounded number of CTAs (eight loads in flight per thread) covers the link and leaves
                # most SMs to the attention kernels
                self._copy(t.data_ptr(), base + self.offsets[j], self._nbytes(j), st, max_ctas=64)
                t.record_stream(self.side)
        ev = torch.cuda.Event()
        ev.record(self.side)
        return out, ev

    def wait_ready(self, src: int, epoch: int) -> None:
        """Make the current stream wait (bounded) until ``src`` has published ``epoch``; kernels enqueued afterwards
        may read ``src``'s slot in place through :meth:`peer_ptr`."""
        self._wait(READY + src, 1, epoch, _native.stream_ptr())

    def peer_ptr(self, src: int, epoch: int, j: int) -> int:
        """Device address, valid in this process, of tensor ``j`` of the payload ``src`` published for ``epoch``."""
        return self.buf.peer_ptrs[src] + (epoch & 1) * self.slot_bytes + self.offsets[j]

    def finish(self, epoch: int) -> None:
        """All pulls of ``epoch`` were consumed on the current stream: let owners reuse the slot."""
        torch.cuda.current_stream(self.device).wait_stream(self.side)
        self._signal(self._ctl_ptrs, self.cp, DONE + self.rank, epoch, _native.stream_ptr())

    # ------------------------------------------------------------------ gradients
    def push_grad(self, owner: int, epoch: int, grads: Sequence[torch.Tensor]) -> None:
        """Deliver fp32 partial gradients of ``owner``'s payload into this rank's partition there."""
        st = _native.stream_ptr()
        if epoch > 2:
            self._wait(GDONE + owner, 1, epoch - 2, st)
        base = self.gbuf.peer_ptrs[owner] + ((epoch & 1) * self.cp + self.rank) * self.g_part_bytes
        for j, g in enumerate(grads):
            g = g.contiguous()
            assert g.dtype == torch.float32 and tuple(g.shape) == self.shapes[j]
            self._copy(base + self.g_offsets[j], g.data_ptr(), g.numel() * 4, st)
        one = (ctypes.c_void_p * 1)(self.ctl.peer_ptrs[owner])
        self._signal(one, 1, GREADY + self.rank, epoch, st)

    def collect_grads(self, epoch: int, local: Sequence[torch.Tensor]) -> List[torch.Tensor]:
        """Sum of the local partial and every peer's delivered partial (rank order), fp32."""
        st = _native.stream_ptr()
        me = (ctypes.c_void_p * 1)(self.ctl.local_ptr)
        self._signal(me, 1, GREADY + self.rank, epoch, st)  # own word, so one wait covers all cp words
        self._wait(GREADY, self.cp, epoch, st)
        out = []
        for j, loc in enumerate(local):
            n = loc.numel()
            acc = None
            for w in range(self.cp):
                if w == self.rank:
                    part = loc
                else:
                    part = self.gbuf.view(((epoch & 1) * self.cp + w) * self.g_part_bytes + self.g_offsets[j], self.shapes[j], torch.float32)
                acc = part.clone() if acc is None else acc.add_(part)
            out.append(acc)
        self._signal(self._ctl_ptrs, self.cp, GDONE + self.rank, epoch, st)
        return out

    def close(self) -> None:
        self.buf.close()
        self.ctl.close()
        if self.with_grads:
            self.gbuf.close()


_EXCHANGES: Dict[tuple, PayloadExchange] = {}


def get_exchange(kind: str, group, cp: int, rank: int, tensors: Sequence[torch.Tensor], with_grads: bool) -> PayloadExchange:
    """Process-wide cache: one exchange per (direction, group, payload signature). Creation is collective."""
    key = (kind, id(group), cp, tuple((tuple(t.shape), t.dtype) for t in tensors))
    ex = _EXCHANGES.get(key)
    if ex is None:
        ex = PayloadExchange(group, cp, rank, [t.shape for t in tensors], [t.dtype for t in tensors], tensors[0].device, with_grads)
        _EXCHANGES[key] = ex
    return ex


def usable(group, cp: int, device) -> bool:
    """CUDA, one node, peer access between all ranks of the group; voted so every rank agrees."""
    import os

    dev = torch.device(device)
    if dev.type != "cuda" or cp <= 1 or cp > 32:
        return False
    from ..contexts import distributed as dctx

    ok = dctx.cp_backend != "nccl"
    local_world = max(int(os.environ.get("LOCAL_WORLD_SIZE", "1")), 1)
    ranks = dist.get_process_group_ranks(group) if group is not None else list(range(dist.get_world_size()))
    me = dist.get_rank()
    ok = ok and all(r // local_world == me // local_world for r in ranks)
    if ok:
        L = _native.lib()
        ok = all(L.pt_can_access_peer(dev.index or 0, r % local_world) == 1 for r in ranks if r != me)
    flag = torch.tensor([1 if ok else 0], dtype=torch.int32, device=dev)
    dist.all_reduce(flag, op=dist.ReduceOp.MIN, group=group)
    return bool(flag.item())
