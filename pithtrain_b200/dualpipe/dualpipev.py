"""DualPipeV scheduler: bidirectional V-shaped pipeline with overlapped forward/backward chunks and
zero-bubble weight phases.

The model is cut into ``2 * pp_size`` stages; rank ``r`` owns stage ``r`` (phase 0) and stage
``2*pp_size-1-r`` (phase 1), so activations flow down the ranks in phase 0 and back up in phase 1
(pithtrain/dualpipe/dualpipev.py:83-111,483-655 of the reference). The order of work on each rank is
data (:func:`pithtrain_b200.dualpipe.schedule.build_schedule`); this module interprets it:
computes chunks with the 5-stage executor, moves activations between ranks with batched
isend/irecv (NCCL on GPUs, gloo on CPU) and defers weight-gradient GEMMs to the W actions through
``WeightGradStore``. The sends of an action's outputs and the receive of the next action's input go
out as one batch at the start of that next action, and the compute stream waits for the batch (the
reference's ``_commit_and_wait_comm`` discipline, which the deadlock simulator of ``schedule.py``
covers); the transfer of one ``(micro_batch, seq/cp, hidden)`` activation is not hidden under
compute.

``step()`` also serves inference: under ``torch.no_grad()`` only forwards run, and
``return_outputs=True`` returns the logits on the rank that owns the last stage (pp rank 0).
"""

from __future__ import annotations

from typing import Callable, List, Optional, Sequence, Tuple

import torch
import torch.distributed as dist
import torch.nn as nn

from ..contexts import distributed
from . import comm
from .execution import ChunkRecord, ExecutionCtx, model_backward, model_forward, nvtx_range
from .overlap import overlapped_forward_backward
from .schedule import Action, backward_dst, backward_src, build_schedule, forward_dst, forward_src
from ..ops.moe import flush_pending_expert_wgrads
from .utils import FP8WeightCacheControl, WeightGradStore, scatter


def layer_partition(num_layers: int, stage_count: int, stage_index: int) -> range:
    """Contiguous block of layer ids owned by ``stage_index``.

    Layers are spread as evenly as possible; surplus layers go to interior stages before the two
    edge stages, which already carry the embedding and the final norm + lm_head (same distribution
    as pithtrain/dualpipe/dualpipev.py:44-62).
    """
    per_stage, surplus = divmod(num_layers, stage_count)
    sizes = [per_stage] * stage_count
    interior = range(1, stage_count - 1)
    for _ in range(surplus):
        low = min(sizes)
        pick = next((i for i in interior if sizes[i] == low), None)
        if pick is None:
            pick = sizes.index(low)
        sizes[pick] += 1
    start = sum(sizes[:stage_index])
    return range(start, start + sizes[stage_index])


class DualPipeV(nn.Module):
    def __init__(self, modules: Sequence[nn.Module], pp_group=None, pp_rank: Optional[int] = None,
                 pp_size: Optional[int] = None) -> None:
        super().__init__()
        assert len(modules) == 2, "DualPipeV drives exactly two model chunks per rank"
        self.module = nn.ModuleList(modules)
        self.group = pp_group if pp_group is not None else distributed.pp_group
        self.pp_rank = distributed.pp_rank if pp_rank is None else pp_rank
        self.pp_size = distributed.pp_size if pp_size is None else pp_size
        self.is_first_rank = self.pp_rank == 0
        self.is_last_rank = self.pp_rank == self.pp_size - 1
        self.comm_stream = None
        if torch.cuda.is_available() and distributed.device.type == "cuda":
            self.comm_stream = torch.cuda.Stream()
        self.overlap = True
        self._reset()

    # ------------------------------------------------------------------ state
    def _reset(self) -> None:
        WeightGradStore.clear()
        self.input_chunks: Tuple[list, list] = ([], [])
        self.output_chunks: Tuple[list, list] = ([], [])
        self.input_grad_chunks: Tuple[list, list] = ([], [])
        self.output_grad_chunks: Tuple[list, list] = ([], [])
        self.records: Tuple[list, list] = ([], [])
        self.labels: Optional[list] = None
        self.loss_chunks: List[torch.Tensor] = []
        self.logit_chunks: List[torch.Tensor] = []
        self.criterion: Optional[Callable] = None
        self.cu_seqlens: Optional[list] = None
        self.f_id = [0, 0]
        self.b_id = [0, 0]
        self.send_f_id = [0, 0]
        self.send_b_id = [0, 0]
        self.comm_ops: list = []
        self.to_free: list = []
        self.forward_only = False
        self.return_outputs = False

    def _record(self, phase: int, chunk_id: int) -> ChunkRecord:
        recs = self.records[phase]
        while len(recs) <= chunk_id:
            recs.append(ChunkRecord(len(self.module[phase].layers)))
        return recs[chunk_id]

    def _is_last_stage(self, phase: int) -> bool:
        return self.is_first_rank and phase == 1

    # ------------------------------------------------------------------ compute
    def _cu(self, chunk_id: int):
        return None if self.cu_seqlens is None else self.cu_seqlens[chunk_id]

    def _finish_forward(self, phase: int, chunk_id: int, out: torch.Tensor) -> None:
        if self._is_last_stage(phase):
            if self.criterion is not None:
                with nvtx_range("criterion"):
                    loss = self.criterion(out, self.labels[chunk_id])
                self.loss_chunks.append(loss)
            if self.return_outputs:
                self.logit_chunks.append(out.detach())
            return
        if self.is_last_rank and phase == 0:
            # hand the activation to the second local chunk without touching the network
            self.input_chunks[1].append(out.detach())
        self.output_chunks[phase].append(out)

    def _forward_compute(self, phase: int) -> None:
        chunk_id = self.f_id[phase]
        self.f_id[phase] += 1
        inputs = self.input_chunks[phase][chunk_id]
        rec = self._record(phase, chunk_id)
        with nvtx_range(f"forward chunk {chunk_id} (phase{phase})"):
            out = model_forward(self.module[phase], inputs, rec, self._cu(chunk_id), ExecutionCtx.make(self.comm_stream))
        if self.forward_only:
            self.input_chunks[phase][chunk_id] = None
            rec.clear()
        self._finish_forward(phase, chunk_id, out)

    def _finish_backward(self, phase: int, chunk_id: int, in_grad: Optional[torch.Tensor]) -> None:
        self.input_chunks[phase][chunk_id] = None
        if not self._is_last_stage(phase):
            self.output_chunks[phase][chunk_id] = None
            self.output_grad_chunks[phase][chunk_id] = None
        if self.is_last_rank and phase == 1:
            self.output_grad_chunks[0].append(in_grad)
        else:
            self.input_grad_chunks[phase].append(in_grad)

    def _backward_inputs(self, phase: int, chunk_id: int):
        if self._is_last_stage(phase):
            loss = self.loss_chunks[chunk_id]
            return None, loss
        return self.output_grad_chunks[phase][chunk_id], None

    def _backward_compute(self, phase: int, enable_zb: bool = False) -> None:
        if self.forward_only:
            return
        chunk_id = self.b_id[phase]
        self.b_id[phase] += 1
        out_grad, loss = self._backward_inputs(phase, chunk_id)
        rec = self._record(phase, chunk_id)
        WeightGradStore.enabled = enable_zb
        try:
            with nvtx_range(f"backward chunk {chunk_id} (phase{phase})"):
                in_grad = model_backward(self.module[phase], rec, out_grad, loss, ExecutionCtx.make(self.comm_stream))
        finally:
            WeightGradStore.enabled = False
        if enable_zb:
            WeightGradStore.flush()
        if loss is not None:
            self.loss_chunks[chunk_id] = loss.detach()
        self._finish_backward(phase, chunk_id, in_grad)

    def _forward_backward_compute(self, phase0: int, phase1: int) -> None:
        if self.forward_only:
            self._forward_compute(phase0)
            return
        if not self.overlap:
            self._forward_compute(phase0)
            self._backward_compute(phase1)
            return
        f_chunk = self.f_id[phase0]
        self.f_id[phase0] += 1
        b_chunk = self.b_id[phase1]
        self.b_id[phase1] += 1
        inputs0 = self.input_chunks[phase0][f_chunk]
        rec0 = self._record(phase0, f_chunk)
        rec1 = self._record(phase1, b_chunk)
        out_grad1, loss1 = self._backward_inputs(phase1, b_chunk)
        with nvtx_range(f"forward chunk {f_chunk} (phase{phase0}) backward chunk {b_chunk} (phase{phase1})"):
            out0, in_grad1 = overlapped_forward_backward(
                self.module[phase0], inputs0, rec0, self._cu(f_chunk),
                self.module[phase1], rec1, out_grad1, loss1, self.comm_stream)
        if loss1 is not None:
            self.loss_chunks[b_chunk] = loss1.detach()
        self._finish_forward(phase0, f_chunk, out0)
        self._finish_backward(phase1, b_chunk, in_grad1)

    def _weight_chunk(self) -> None:
        if self.forward_only:
            return
        self._commit_and_wait_comm()
        with nvtx_range("weight chunk"):
            WeightGradStore.pop()

    # ------------------------------------------------------------------ communication
    def _recv_forward(self, phase: int) -> None:
        src = forward_src(self.pp_size, self.pp_rank, phase)
        if src is None:
            return
        tensors = comm.append_irecv(self.comm_ops, src, self.group, distributed.device)
        self.input_chunks[phase].append(tensors[0].detach())

    def _send_forward(self, phase: int) -> None:
        dst = forward_dst(self.pp_size, self.pp_rank, phase)
        if dst is None:
            return
        chunk_id = self.send_f_id[phase]
        self.send_f_id[phase] += 1
        comm.append_isend(self.comm_ops, [self.output_chunks[phase][chunk_id]], dst, self.group)
        if self.forward_only:
            self.output_chunks[phase][chunk_id] = None

    def _recv_backward(self, phase: int) -> None:
        if self.forward_only:
            return
        src = backward_src(self.pp_size, self.pp_rank, phase)
        if src is None:
            return
        tensors = comm.append_irecv(self.comm_ops, src, self.group, distributed.device)
        self.output_grad_chunks[phase].append(tensors[0].detach())

    def _send_backward(self, phase: int) -> None:
        if self.forward_only:
            return
        dst = backward_dst(self.pp_size, self.pp_rank, phase)
        if dst is None:
            return
        chunk_id = self.send_b_id[phase]
        self.send_b_id[phase] += 1
        g = self.input_grad_chunks[phase][chunk_id]
        self.input_grad_chunks[phase][chunk_id] = None
        comm.append_isend(self.comm_ops, [g], dst, self.group)

    def _commit_and_wait_comm(self) -> None:
        if not self.comm_ops:
            return
        with nvtx_range("pipeline send/recv"):
            reqs = dist.batch_isend_irecv(self.comm_ops)
            for r in reqs:
                r.wait()
        self.comm_ops = []

    # ------------------------------------------------------------------ actions
    def _run(self, a: Action) -> None:
        k = a.kind
        if k == "RECV_F":
            self._recv_forward(a.phase)
        elif k == "SEND_F":
            self._send_forward(a.phase)
        elif k == "SEND_B":
            self._send_backward(a.phase)
        elif k == "F":
            if a.recv:
                self._recv_forward(a.phase)
            self._commit_and_wait_comm()
            self._forward_compute(a.phase)
            if a.send:
                self._send_forward(a.phase)
        elif k == "B":
            if self.forward_only:
                return
            if a.recv:
                self._recv_backward(a.phase)
            self._commit_and_wait_comm()
            self._backward_compute(a.phase, enable_zb=a.zb)
            if a.send:
                self._send_backward(a.phase)
        elif k == "FB":
            if a.recv:
                self._recv_forward(a.phase)
            self._recv_backward(a.bphase)
            self._commit_and_wait_comm()
            self._forward_backward_compute(a.phase, a.bphase)
            self._send_forward(a.phase)
            self._send_backward(a.bphase)
        elif k == "W":
            self._weight_chunk()
        else:
            raise ValueError(k)

    # ------------------------------------------------------------------ public
    def setup_cu_seqlens(self, cu_seqlens, num_chunks: int):
        """Broadcast per-micro-batch document offsets from pipeline rank 0 to the other pp ranks."""
        if self.pp_size == 1 or not dist.is_initialized():
            return cu_seqlens
        dev = distributed.device
        width = torch.zeros(1, dtype=torch.int64, device=dev)
        if self.is_first_rank and cu_seqlens is not None:
            width[0] = max(int(c.numel()) for c in cu_seqlens)
        src = dist.get_global_rank(self.group, 0)
        dist.broadcast(width, src=src, group=self.group)
        w = int(width.item())
        if w == 0:
            return None
        table = torch.full((num_chunks, w), -1, dtype=torch.int32, device=dev)
        if self.is_first_rank:
            for i, c in enumerate(cu_seqlens):
                table[i, : c.numel()] = c.to(torch.int32)
        dist.broadcast(table, src=src, group=self.group)
        return [row[row >= 0] for row in table]

    def step(self, *inputs: Optional[torch.Tensor], num_chunks: int = 0, criterion: Optional[Callable] = None,
             labels: Optional[torch.Tensor] = None, cu_seqlens: Optional[list] = None, return_outputs: bool = False):
        """Run ``num_chunks`` micro-batches through the pipeline (forward and, unless grad is
        disabled, backward). ``inputs``/``labels`` are needed on pipeline rank 0 only.

        Returns ``(loss, outputs)``: per-micro-batch losses stacked (pp rank 0, else ``None``) and
        the concatenated last-stage outputs when ``return_outputs``.
        """
        assert num_chunks >= 2 * self.pp_size, f"num_chunks ({num_chunks}) must be >= 2 * pp_size"
        self._reset()
        self.forward_only = not torch.is_grad_enabled()
        self.return_outputs = return_outputs
        self.criterion = criterion
        FP8WeightCacheControl.step()
        if self.is_first_rank:
            assert inputs and inputs[0] is not None, "pipeline rank 0 needs the input token ids"
            self.input_chunks = ([m[0] for m in scatter(inputs[0], num_chunks, 0)], [])
            if labels is not None:
                self.labels = [m[0] for m in scatter(labels, num_chunks, 0)]
        self.cu_seqlens = self.setup_cu_seqlens(cu_seqlens, num_chunks)

        for action in build_schedule(self.pp_size, self.pp_rank, num_chunks):
            self._run(action)
        assert not WeightGradStore.funcs_queue, "deferred weight gradients left in the queue"
        flush_pending_expert_wgrads()
        self._commit_and_wait_comm()

        loss, outputs = None, None
        if self.is_first_rank:
            if self.loss_chunks:
                loss = torch.stack([x.detach() for x in self.loss_chunks])
            if return_outputs and self.logit_chunks:
                outputs = torch.cat(self.logit_chunks, dim=0)
        FP8WeightCacheControl.clear(*self.module)
        self._reset()
        return loss, outputs

    def forward(self, *args, **kwargs):  # pragma: no cover - nn.Module plumbing
        return self.step(*args, **kwargs)
