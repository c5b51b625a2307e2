"""Shard-group collectives as kernels over peer memory (the CUDA side is ``csrc/fsdp_fused.cu``).

``FusedShardComm`` owns three symmetric allocations of one flat shard group — parameters, gradient
accumulators, a small control block — and drives the step protocol:

    backward ...                      gradients accumulate in the local flat buffer
    reduce_scatter(scale)             flag "final"; owner sums its region over all peers' buffers,
                                      averages, writes it locally and returns sum(g^2) partials
    optimizer on the owned region
    push_params()                     owner stores its region into every peer's parameter buffer
    before_zero_grad()                wait until every owner finished reading this rank's gradients
    before_forward()                  wait until all regions were published

No NCCL call is involved; a rank only ever blocks inside bounded in-kernel waits that report through
the library's status word. All ranks of the group must be on one node with peer access.
"""

from __future__ import annotations

import ctypes


import torch
import torch.distributed as dist

from .. import _native
from .symm_mem import SymmetricBuffer

MAXW = 32


class FsdpChanStruct(ctypes.Structure):
    _fields_ = [("W", ctypes.c_int), ("rank", ctypes.c_int), ("fp32", ctypes.c_int), ("region", ctypes.c_longlong),
                ("grad", ctypes.c_void_p * MAXW), ("param", ctypes.c_void_p * MAXW), ("ctl", ctypes.c_void_p * MAXW),
                ("param_bytes", ctypes.c_int)]


class FusedShardComm:
    def __init__(self, group, group_size: int, group_rank: int, region: int, param_dtype: torch.dtype,
                 grad_dtype: torch.dtype, device) -> None:
        assert 1 < group_size <= MAXW
        assert grad_dtype in (torch.float32, torch.bfloat16)
        L = _native.lib()
        self.group, self.W, self.rank, self.region = group, group_size, group_rank, region
        total = region * group_size
        pbytes = torch.empty((), dtype=param_dtype).element_size()
        gbytes = torch.empty((), dtype=grad_dtype).element_size()
        self.param_buf = SymmetricBuffer(total * pbytes, group, device, "shard parameters")
        self.grad_buf = SymmetricBuffer(total * gbytes, group, device, "shard gradients")
        self.ctl_buf = SymmetricBuffer(L.pt_fsdp_ctl_bytes(), group, device, "shard control")
        self.flat_param = self.param_buf.view(0, (total,), param_dtype)
        self.flat_grad = self.grad_buf.view(0, (total,), grad_dtype)
        s = FsdpChanStruct()
        s.W, s.rank, s.fp32, s.region, s.param_bytes = group_size, group_rank, int(grad_dtype == torch.float32), region, pbytes
        for r in range(group_size):
            s.grad[r], s.param[r], s.ctl[r] = self.grad_buf.peer_ptrs[r], self.param_buf.peer_ptrs[r], self.ctl_buf.peer_ptrs[r]
        assert ctypes.sizeof(s) == L.pt_fsdp_chan_struct_size(), "fsdp Chan layout mismatch"
        self.struct, self.cptr = s, ctypes.addressof(s)
        self.epoch = 0  # reduce-scatter rounds
        self.push_epoch = 0
        self._partials = torch.zeros(L.pt_fsdp_reduce_grid(), dtype=torch.float64, device=device)
        self._acks_pending = False
        self._params_pending = False

    # ------------------------------------------------------------------ gradients
    def reduce_scatter(self, scale: float = 1.0) -> torch.Tensor:
        """Average this rank's region over the group (in place); returns sum(g^2) of the result."""
        L, st = _native.lib(), _native.stream_ptr()
        self.epoch += 1
        _native.check(L.pt_fsdp_signal_ready(self.cptr, self.epoch, st), "pt_fsdp_signal_ready")
        rc = L.pt_fsdp_reduce_scatter(self.cptr, self.epoch, float(scale) / self.W, self._partials.data_ptr(), st)
        _native.check(rc, "pt_fsdp_reduce_scatter")
        self._acks_pending = True
        return self._partials.sum().float()

    def before_zero_grad(self) -> None:
        if self._acks_pending:
            _native.check(_native.lib().pt_fsdp_wait_acks(self.cptr, self.epoch, _native.stream_ptr()), "pt_fsdp_wait_acks")
            self._acks_pending = False

    # ------------------------------------------------------------------ parameters
    def push_params(self) -> None:
        self.push_epoch += 1
        rc = _native.lib().pt_fsdp_push_params(self.cptr, self.push_epoch, _native.stream_ptr())
        _native.check(rc, "pt_fsdp_push_params")
        self._params_pending = True

    def before_forward(self) -> None:
        if self._params_pending:
            rc = _native.lib().pt_fsdp_wait_params(self.cptr, self.push_epoch, _native.stream_ptr())
            _native.check(rc, "pt_fsdp_wait_params")
            self._params_pending = False

    def close(self) -> None:
        for b in (self.param_buf, self.grad_buf, self.ctl_buf):
            b.close()


def usable(group, group_size: int, device) -> bool:
    """Whether a shard group can use the peer-memory collectives: CUDA, one node, peer access; voted."""
    import os

    dev = torch.device(device)
    if dev.type != "cuda" or group_size <= 1 or group_size > MAXW:
        return False
    from ..contexts import distributed as dctx

    ok = dctx.shard_backend != "nccl"
    local_world = int(os.environ.get("LOCAL_WORLD_SIZE", "1"))
    ranks = dist.get_process_group_ranks(group)
    me_global = dist.get_rank()
    node = me_global // max(local_world, 1)
    ok = ok and all(r // max(local_world, 1) == node for r in ranks)
    if ok:
        L = _native.lib()
        me = dev.index or 0
        ok = all(L.pt_can_access_peer(me, r % local_world) == 1 for r in ranks if r != me_global)
    flag = torch.tensor([1 if ok else 0], dtype=torch.int32, device=dev)
    dist.all_reduce(flag, op=dist.ReduceOp.MIN, group=group)
    return bool(flag.item())
