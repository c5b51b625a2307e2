"""Fused expert-parallel transport: dispatch and combine as kernels that read and write peer memory.

Same contract as :class:`pithtrain_b200.parallel.ep.CollectiveExchange`, but

* the send plan is one kernel and stays on the device (no ``nonzero``, no count read-back);
* dispatch gathers each de-duplicated row by index and stores it straight into the destination
  rank's partition of a symmetric buffer over NVLink, with the row's local expert ids and routing
  weights riding along; the receiver compacts the partitions into a dense tensor whose length is a
  device-side count;
* combine writes every partial row back into the cell it came from, and the home rank sums a
  token's cells in the same launch sequence, so combine already returns ``[tokens, hidden]``;
* backward of each direction is the other direction over the same plan.

Four channels (dispatch/combine × forward/backward), two slots each, sized once from the first
micro-batch shape. Receive capacity is the exact worst case (every token of every rank routed here,
``ep * m`` rows) unless ``capacity_factor`` is given explicitly, in which case it is that multiple of the
expected de-duplicated volume: an opt-in that saves memory for well-balanced routers. An overflow of a reduced
capacity sets the status word, which the train step reads once per step and turns into an error on every rank.
"""

from __future__ import annotations

import ctypes
from typing import Dict, Tuple

import torch

from .. import _native
from ..ops.moe import combine_rows
from .ep import DispatchPlan, Exchange
from .symm_mem import SymmetricBuffer

EP_MAX = 32


class EpChanStruct(ctypes.Structure):
    _fields_ = [("ep", ctypes.c_int), ("rank", ctypes.c_int), ("cap", ctypes.c_int), ("W", ctypes.c_int),
                ("k", ctypes.c_int), ("off_data", ctypes.c_longlong), ("off_mi", ctypes.c_longlong),
                ("off_mf", ctypes.c_longlong), ("off_count", ctypes.c_longlong), ("off_flag", ctypes.c_longlong),
                ("off_ack", ctypes.c_longlong), ("off_done", ctypes.c_longlong), ("base", ctypes.c_void_p * EP_MAX)]


def _align(n: int, a: int = 256) -> int:
    return (n + a - 1) // a * a


class Channel:
    """One direction of traffic: symmetric buffer + epoch bookkeeping."""

    def __init__(self, group, ep: int, rank: int, cap: int, row_bytes: int, k: int, device):
        self.ep, self.rank, self.cap, self.W, self.k = ep, rank, cap, row_bytes, k
        cells = 2 * ep * cap
        off = 0
        self.off_data = off; off = _align(off + cells * row_bytes)
        self.off_mi = off; off = _align(off + cells * max(k, 1) * 4)
        self.off_mf = off; off = _align(off + cells * max(k, 1) * 4)
        self.off_count = off; off = _align(off + 2 * ep * 4)
        self.off_flag = off; off = _align(off + 2 * ep * 4)
        self.off_ack = off; off = _align(off + 2 * ep * 4)
        self.off_done = off; off = _align(off + 64)
        self.buf = SymmetricBuffer(off, group, device, "expert-parallel channel")
        s = EpChanStruct()
        s.ep, s.rank, s.cap, s.W, s.k = ep, rank, cap, row_bytes, k
        s.off_data, s.off_mi, s.off_mf = self.off_data, self.off_mi, self.off_mf
        s.off_count, s.off_flag, s.off_ack, s.off_done = self.off_count, self.off_flag, self.off_ack, self.off_done
        for r in range(ep):
            s.base[r] = self.buf.peer_ptrs[r]
        assert ctypes.sizeof(s) == _native.lib().pt_ep_chan_struct_size(), "EpChan layout mismatch"
        self.struct = s
        self.cptr = ctypes.addressof(s)
        self.done_ptr = self.buf.local_ptr + self.off_done
        self.epoch = 0

    def next(self) -> Tuple[int, int]:
        self.epoch += 1
        return self.epoch, self.epoch & 1

    def data_view(self, slot: int, dtype=torch.bfloat16) -> torch.Tensor:
        es = torch.empty((), dtype=dtype).element_size()
        n = self.ep * self.cap
        return self.buf.view(self.off_data + slot * n * self.W, (n, self.W // es), dtype)

    def mf_view(self, slot: int) -> torch.Tensor:
        n = self.ep * self.cap
        return self.buf.view(self.off_mf + slot * n * self.k * 4, (n, self.k), torch.float32)


class _FusedDispatch(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, plan, ex):
        L = _native.lib()
        ch = ex.channels["dispatch_f"]
        epoch, slot = ch.next()
        x = x.contiguous()
        wf = w.detach().float().contiguous()
        st = _native.stream_ptr()
        rc = L.pt_ep_push(ch.cptr, slot, epoch, x.data_ptr(), x.stride(0) * x.element_size(),
                          plan.send_token_idx.data_ptr(), plan.counts_dev.data_ptr(), plan.send_eids.data_ptr(),
                          wf.data_ptr(), ch.done_ptr, st)
        _native.check(rc, "pt_ep_push")
        dev, H, k, cap_total = x.device, x.shape[1], plan.k, ex.cap_total
        recv_x = torch.empty((cap_total, H), dtype=x.dtype, device=dev)
        recv_eids = torch.empty((cap_total, k), dtype=torch.int32, device=dev)
        recv_w = torch.empty((cap_total, k), dtype=torch.float32, device=dev)
        prefix = torch.empty(plan.ep + 1, dtype=torch.int32, device=dev)
        rc = L.pt_ep_receive(ch.cptr, slot, epoch, prefix.data_ptr(), recv_x.data_ptr(), recv_eids.data_ptr(),
                             recv_w.data_ptr(), cap_total, st)
        _native.check(rc, "pt_ep_receive")
        plan.recv_eids, plan.recv_prefix = recv_eids, prefix
        plan.n_recv_dev = prefix[plan.ep:plan.ep + 1]
        ctx.plan, ctx.ex, ctx.w_dtype = plan, ex, w.dtype
        return recv_x, recv_w

    @staticmethod
    def backward(ctx, d_recv_x, d_recv_w):
        L = _native.lib()
        plan, ex = ctx.plan, ctx.ex
        ch = ex.channels["dispatch_b"]
        epoch, slot = ch.next()
        st = _native.stream_ptr()
        d_recv_x = d_recv_x.contiguous()
        dw_rows = torch.zeros((ex.cap_total, plan.k), dtype=torch.float32, device=d_recv_x.device) \
            if d_recv_w is None else d_recv_w.float().contiguous()
        rc = L.pt_ep_return(ch.cptr, slot, epoch, d_recv_x.data_ptr(), dw_rows.data_ptr(), plan.recv_prefix.data_ptr(),
                            ch.done_ptr, st)
        _native.check(rc, "pt_ep_return")
        _native.check(L.pt_ep_wait_returned(ch.cptr, slot, epoch, st), "pt_ep_wait_returned")
        pos = plan.token_send_pos
        d_x = combine_rows(ch.data_view(slot, d_recv_x.dtype), pos.reshape(-1), plan.ep)
        mf = ch.mf_view(slot)
        mf_ext = torch.cat([mf, mf.new_zeros(1, plan.k)])
        d_w = mf_ext[pos.long()].sum(1).to(ctx.w_dtype)  # -1 picks the appended zero row
        _native.check(L.pt_ep_ack(ch.cptr, slot, epoch, st), "pt_ep_ack")
        return d_x, d_w, None, None


class _FusedCombine(torch.autograd.Function):
    @staticmethod
    def forward(ctx, partial, plan, ex):
        L = _native.lib()
        ch = ex.channels["combine_f"]
        epoch, slot = ch.next()
        st = _native.stream_ptr()
        partial = partial.contiguous()
        rc = L.pt_ep_return(ch.cptr, slot, epoch, partial.data_ptr(), None, plan.recv_prefix.data_ptr(), ch.done_ptr, st)
        _native.check(rc, "pt_ep_return")
        _native.check(L.pt_ep_wait_returned(ch.cptr, slot, epoch, st), "pt_ep_wait_returned")
        out = combine_rows(ch.data_view(slot, partial.dtype), plan.token_send_pos.reshape(-1), plan.ep)
        _native.check(L.pt_ep_ack(ch.cptr, slot, epoch, st), "pt_ep_ack")
        ctx.plan, ctx.ex = plan, ex
        return out

    @staticmethod
    def backward(ctx, d_out):
        L = _native.lib()
        plan, ex = ctx.plan, ctx.ex
        ch = ex.channels["combine_b"]
        epoch, slot = ch.next()
        st = _native.stream_ptr()
        d_out = d_out.contiguous()
        rc = L.pt_ep_push(ch.cptr, slot, epoch, d_out.data_ptr(), d_out.stride(0) * d_out.element_size(),
                          plan.send_token_idx.data_ptr(), plan.counts_dev.data_ptr(), None, None, ch.done_ptr, st)
        _native.check(rc, "pt_ep_push")
        d_partial = torch.empty((ex.cap_total, d_out.shape[1]), dtype=d_out.dtype, device=d_out.device)
        prefix = torch.empty(plan.ep + 1, dtype=torch.int32, device=d_out.device)
        rc = L.pt_ep_receive(ch.cptr, slot, epoch, prefix.data_ptr(), d_partial.data_ptr(), None, None, ex.cap_total, st)
        _native.check(rc, "pt_ep_receive")
        return d_partial, None, None


class FusedExchange(Exchange):
    def __init__(self, group, ep_size: int, ep_rank: int, capacity_factor: float | None = None) -> None:
        assert ep_size <= EP_MAX
        self.group, self.ep, self.rank = group, ep_size, ep_rank
        self.capacity_factor = capacity_factor
        self.channels: Dict[str, Channel] = {}
        self.cap = 0
        self.cap_total = 0

    def _ensure_channels(self, m: int, H: int, k: int, device, elem_size: int = 2) -> None:
        if self.channels:
            assert m <= self.cap, f"micro-batch of {m} tokens exceeds the exchange capacity {self.cap}"
            return
        self.cap = m
        worst = self.ep * m
        self.cap_total = worst
        if self.capacity_factor is not None:
            expected = self.ep * m * (1.0 - ((self.ep - 1) / self.ep) ** k)
            want = int(self.capacity_factor * expected) + m
            self.cap_total = min(worst, (want + 127) // 128 * 128)
        W = H * elem_size
        for name, kk in (("dispatch_f", k), ("dispatch_b", k), ("combine_f", 0), ("combine_b", 0)):
            self.channels[name] = Channel(self.group, self.ep, self.rank, m, W, kk, device)

    def plan(self, topk_idx: torch.Tensor, num_experts: int) -> DispatchPlan:
        m, k = topk_idx.shape
        dev = topk_idx.device
        self._plan_shape = (m, k)
        idx = topk_idx.int().contiguous()
        cap = self.cap or m
        pos = torch.empty((m, self.ep), dtype=torch.int32, device=dev)
        send_token_idx = torch.empty(self.ep * cap, dtype=torch.int32, device=dev)
        send_eids = torch.empty((self.ep * cap, k), dtype=torch.int32, device=dev)
        counts = torch.empty(self.ep, dtype=torch.int32, device=dev)
        rc = _native.lib().pt_ep_plan(idx.data_ptr(), m, k, num_experts // self.ep, self.ep, cap, pos.data_ptr(),
                                      send_token_idx.data_ptr(), send_eids.data_ptr(), counts.data_ptr(),
                                      _native.stream_ptr())
        _native.check(rc, "pt_ep_plan")
        plan = DispatchPlan(m=m, k=k, ep=self.ep, send_token_idx=send_token_idx, token_send_pos=pos,
                            send_eids=send_eids, send_counts=[], recv_counts=[])
        plan.counts_dev = counts
        plan.reduced = True
        return plan

    def dispatch(self, x, w, plan):
        self._ensure_channels(x.shape[0], x.shape[1], plan.k, x.device, x.element_size())
        return _FusedDispatch.apply(x, w, plan, self)

    def combine(self, partial, plan):
        return _FusedCombine.apply(partial, plan, self)

    def close(self) -> None:
        for ch in self.channels.values():
            ch.buf.close()
        self.channels = {}
