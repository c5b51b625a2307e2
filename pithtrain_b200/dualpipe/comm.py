"""Pipeline point-to-point traffic: one pending batch of isend/irecv operations per executor.

Everything that crosses a pipeline boundary — an activation going down, a gradient coming back — has the same
static signature ``(micro_batch, seq/cp, hidden)`` in the compute dtype. The signature is published once per job
(:func:`set_p2p_tensor_shapes`, :func:`set_p2p_tensor_dtype`; the setter names are those of the reference,
pithtrain/dualpipe/comm.py:14-25, because user code calls them). :class:`P2PBatch` collects the operations an
executor posts between two compute actions and commits them as one ``batch_isend_irecv``.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import List, Sequence, Tuple

import torch
import torch.distributed as dist


@dataclass
class _Signature:
    shapes: List[Tuple[int, ...]] = field(default_factory=list)
    dtype: torch.dtype = torch.bfloat16


SIGNATURE = _Signature()


def set_p2p_tensor_shapes(shapes: Sequence[Tuple[int, ...]]) -> None:
    SIGNATURE.shapes = [tuple(s) for s in shapes]


def set_p2p_tensor_dtype(dtype: torch.dtype) -> None:
    SIGNATURE.dtype = dtype


def _global_rank(group, rank_in_group: int) -> int:
    return rank_in_group if group is None else dist.get_global_rank(group, rank_in_group)


class P2PBatch:
    """Operations waiting for the next commit. ``recv`` hands out the landing buffers immediately; they are valid
    after :meth:`commit`."""

    def __init__(self, group, device) -> None:
        self.group, self.device = group, device
        self.ops: List[dist.P2POp] = []

    def __bool__(self) -> bool:
        return bool(self.ops)

    def recv(self, src: int) -> List[torch.Tensor]:
        peer = _global_rank(self.group, src)
        landing = [torch.empty(shape, dtype=SIGNATURE.dtype, device=self.device, requires_grad=True) for shape in SIGNATURE.shapes]
        self.ops.extend(dist.P2POp(dist.irecv, t, peer, self.group) for t in landing)
        return landing

    def send(self, tensors: Sequence[torch.Tensor], dst: int) -> None:
        peer = _global_rank(self.group, dst)
        self.ops.extend(dist.P2POp(dist.isend, t.detach().contiguous(), peer, self.group) for t in tensors)

    def commit(self) -> None:
        """Issue everything posted so far as one batch and wait for it."""
        if not self.ops:
            return
        for req in dist.batch_isend_irecv(self.ops):
            req.wait()
        self.ops = []


# function-style spellings used by older call sites
def append_irecv(ops: list, src: int, group, device) -> List[torch.Tensor]:
    batch = P2PBatch(group, device)
    out = batch.recv(src)
    ops.extend(batch.ops)
    return out


def append_isend(ops: list, tensors: Sequence[torch.Tensor], dst: int, group) -> None:
    batch = P2PBatch(group, None)
    batch.send(tensors, dst)
    ops.extend(batch.ops)
