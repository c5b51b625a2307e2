"""Symmetric memory: one buffer per rank of a process group, mapped into every rank.

``SymmetricBuffer(nbytes, group)`` allocates ``nbytes`` on this rank (cudaMalloc inside the native
library), exchanges CUDA IPC handles over the group and opens every peer's allocation, so kernels
can address ``peer_ptrs[r]`` directly over NVLink. ``view(offset, shape, dtype)`` exposes parts of
the local buffer as torch tensors (zero-copy, through the CUDA array interface) so ordinary ops
and kernels can consume received data in place. All ranks of the group must be on one node.

Every allocation ends in a guard region of ``GUARD_BYTES`` filled with a fixed pattern that no kernel
is ever given as part of its extent. Peers write into these buffers with plain stores over NVLink, so
an index error on another GPU would otherwise corrupt whatever follows silently;
:meth:`SymmetricBuffer.check_guard` (called when the buffer is closed, and by ``check_all_guards`` at
checkpoint time and from tests) turns such an overrun into an error that names the buffer.
"""

from __future__ import annotations

import ctypes
from typing import List, Sequence

import torch
import torch.distributed as dist

from .. import _native


class _RawCuda:
    """Adapter that lets ``torch.as_tensor`` wrap a raw device pointer."""

    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 2}


GUARD_BYTES = 4096
GUARD_WORD = 0x5AA55AA5
_LIVE: "List[SymmetricBuffer]" = []


class GuardOverrun(RuntimeError):
    """A kernel wrote past the end of a symmetric buffer."""


def check_all_guards() -> None:
    """Verify the guard region of every live symmetric buffer of this process (a few 4 KB device-to-host copies)."""
    for b in list(_LIVE):
        b.check_guard()


class SymmetricBuffer:
    def __init__(self, nbytes: int, group, device: torch.device, name: str = ""):
        L = _native.lib()
        self.group, self.device, self.name = group, device, name
        self.nbytes = (int(nbytes) + 255) // 256 * 256
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        out = ctypes.c_void_p()
        with torch.cuda.device(device):
            rc = L.pt_symm_malloc(ctypes.addressof(out), self.nbytes + GUARD_BYTES)
        _native.check(rc, "pt_symm_malloc")
        self.local_ptr = int(out.value)
        hsize = L.pt_ipc_handle_size()
        handle = (ctypes.c_ubyte * hsize)()
        _native.check(L.pt_ipc_export(self.local_ptr, ctypes.addressof(handle)), "pt_ipc_export")
        handles: List[bytes] = [b""] * self.world
        dist.all_gather_object(handles, bytes(handle), group=group)
        self.peer_ptrs: List[int] = []
        self._opened: List[int] = []
        for r, h in enumerate(handles):
            if r == self.rank:
                self.peer_ptrs.append(self.local_ptr)
                continue
            buf = (ctypes.c_ubyte * hsize).from_buffer_copy(h)
            p = ctypes.c_void_p()
            with torch.cuda.device(device):
                rc = L.pt_ipc_import(ctypes.addressof(buf), ctypes.addressof(p))
            _native.check(rc, "pt_ipc_import")
            self.peer_ptrs.append(int(p.value))
            self._opened.append(int(p.value))
        self._raw = torch.as_tensor(_RawCuda(self.local_ptr, self.nbytes), device=device)
        self._guard = torch.as_tensor(_RawCuda(self.local_ptr + self.nbytes, GUARD_BYTES), device=device).view(torch.int32)
        self._guard.fill_(GUARD_WORD - (1 << 32) if GUARD_WORD >= (1 << 31) else GUARD_WORD)
        torch.cuda.synchronize(device)
        _LIVE.append(self)
        dist.barrier(group=group)

    def check_guard(self) -> None:
        """Raise :class:`GuardOverrun` if anything wrote into the guard region behind this rank's allocation."""
        if not self.local_ptr:
            return
        want = GUARD_WORD - (1 << 32) if GUARD_WORD >= (1 << 31) else GUARD_WORD
        bad = (self._guard != want).nonzero()
        if bad.numel():
            first = int(bad[0])
            raise GuardOverrun(f"symmetric buffer {self.name or hex(self.local_ptr)} ({self.nbytes} bytes) of rank {self.rank}: "
                               f"{bad.numel()} guard words overwritten, first at byte {self.nbytes + 4 * first}")

    def view(self, offset: int, shape: Sequence[int], dtype: torch.dtype) -> torch.Tensor:
        n = 1
        for s in shape:
            n *= int(s)
        nbytes = n * torch.empty((), dtype=dtype).element_size()
        assert offset % 16 == 0 and offset + nbytes <= self.nbytes
        return self._raw[offset:offset + nbytes].view(dtype).view(*shape)

    def close(self) -> None:
        L = _native.lib()
        if self in _LIVE:
            _LIVE.remove(self)
        self.check_guard()
        for p in self._opened:
            L.pt_ipc_close(p)
        self._opened = []
        if self.local_ptr:
            L.pt_symm_free(self.local_ptr)
            self.local_ptr = 0
