"""Pipeline point-to-point helpers (NCCL/gloo isend-irecv batches).

Activations and their gradients travelling between pipeline stages all have one static shape
``(micro_batch, seq/cp, hidden)``, published once through :func:`set_p2p_tensor_shapes`
(same contract as pithtrain/dualpipe/comm.py:14-49).
"""

from __future__ import annotations

from typing import List, Tuple

import torch
import torch.distributed as dist

TENSOR_SHAPES: List[Tuple[int, ...]] = []
TENSOR_DTYPE: torch.dtype = torch.bfloat16


def set_p2p_tensor_shapes(shapes: List[Tuple[int, ...]]) -> None:
    global TENSOR_SHAPES
    TENSOR_SHAPES = list(shapes)


def set_p2p_tensor_dtype(dtype: torch.dtype) -> None:
    global TENSOR_DTYPE
    TENSOR_DTYPE = dtype


def build_from_tensor_shapes(device) -> List[torch.Tensor]:
    return [torch.empty(s, dtype=TENSOR_DTYPE, device=device, requires_grad=True) for s in TENSOR_SHAPES]


def append_irecv(ops: list, src: int, group, device) -> List[torch.Tensor]:
    tensors = build_from_tensor_shapes(device)
    src = dist.get_global_rank(group, src) if group is not None else src
    for t in tensors:
        ops.append(dist.P2POp(dist.irecv, t, src, group))
    return tensors


def append_isend(ops: list, tensors: List[torch.Tensor], dst: int, group) -> None:
    dst = dist.get_global_rank(group, dst) if group is not None else dst
    for t in tensors:
        ops.append(dist.P2POp(dist.isend, t.detach().contiguous(), dst, group))
