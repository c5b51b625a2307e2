"""Block-scaled e4m3 casts with the names and output shapes of the reference's quantiser wrappers
(pithtrain/operators/deepgemm_quantize.py:204-899), built on this package's two kernels
(:func:`pithtrain_b200.ops.quant.quant_rows`: 1x128 row segments; :func:`pithtrain_b200.ops.quant.quant_blocks`:
128x128 tiles, both orientations in one pass). The scale rule is the same power-of-two rule, so payloads and scales
are equal to the reference's bit for bit; what differs is the fusion: a "row + column" cast here is two passes.

The training path does not call these (it quantises inside :mod:`pithtrain_b200.ops.fp8_linear`); they serve code
written against the reference's operator module.
"""
from __future__ import annotations

from typing import Tuple

import torch

from .quant import quant_blocks, quant_rows

__all__ = ["fp8cast_rowwise_colwise", "fp8cast_rowwise_kmajor", "fp8cast_rowwise_transpose",
           "fp8cast_rowwise_blockwise_transpose", "fp8cast_blockwise_transpose", "fp8cast_blockwise_transpose_batched"]

Four = Tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor]


def _rows(x: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """``(q [M, N], scale [M, ceil(N/128)])`` — the row-major scale layout of the reference."""
    q, s = quant_rows(x.contiguous())
    return q, s[:, :x.shape[0]].t().contiguous()


def fp8cast_rowwise_colwise(x: torch.Tensor) -> Four:
    """``(tok_fp8 [M,N], tok_scale [M, ceil(N/128)], ch_fp8 [M,N], ch_scale [M/128, N])``; ``M % 128 == 0``."""
    assert x.ndim == 2 and x.shape[0] % 128 == 0, f"expected 2-D with M % 128 == 0, got {tuple(x.shape)}"
    tok, tok_s = _rows(x)
    qt, st = quant_rows(x.t().contiguous())  # column segments of x are row segments of x^T
    return tok, tok_s, qt.t().contiguous(), st[:, :x.shape[1]].contiguous()


def fp8cast_rowwise_kmajor(x: torch.Tensor, grouped_mm_offs: torch.Tensor) -> Four:
    """Row-wise cast plus the column-wise payload laid out group by group as ``[N, rows_g]`` blocks in one flat
    ``[M * N]`` tensor, with the column-wise scales transposed to ``[N, M/128]`` (the reference's grouped-wgrad operand).
    ``grouped_mm_offs`` holds the cumulative row counts; rows past the last one (if any) form a trailing block.
    Nothing is read back to the host: the destination of every element is computed on the device."""
    tok, tok_s, ch, ch_s = fp8cast_rowwise_colwise(x)
    M, N = x.shape
    offs = grouped_mm_offs.to(device=x.device, dtype=torch.int64)
    rows = torch.arange(M, device=x.device, dtype=torch.int64)
    ends = torch.cat([offs, torch.full((1,), M, device=x.device, dtype=torch.int64)])
    g = torch.searchsorted(ends, rows, right=True)            # block of every row
    starts = torch.cat([torch.zeros(1, device=x.device, dtype=torch.int64), ends])[g]
    lens = ends[g.clamp(max=ends.numel() - 1)] - starts
    # element (r, n) of block [start, start + len) goes to start * N + n * len + (r - start)
    dest = (starts * N + rows - starts).unsqueeze(1) + torch.arange(N, device=x.device, dtype=torch.int64).unsqueeze(0) * lens.unsqueeze(1)
    flat = torch.empty(M * N, dtype=torch.uint8, device=x.device)
    flat[dest.reshape(-1)] = ch.view(torch.uint8).reshape(-1)
    return tok, tok_s, flat.view(torch.float8_e4m3fn), ch_s.t().contiguous()


def fp8cast_rowwise_transpose(x: torch.Tensor) -> Four:
    """``(tok_fp8 [M,N], tok_scale [M, ceil(N/128)], t_fp8 [N,M], t_scale [N, ceil(M/128)])``."""
    assert x.ndim == 2
    tok, tok_s = _rows(x)
    t, t_s = _rows(x.t())
    return tok, tok_s, t, t_s


def fp8cast_rowwise_blockwise_transpose(x: torch.Tensor) -> Four:
    """``(tok_fp8 [M,K], tok_scale [M, ceil(K/128)], blk_t_fp8 [K,M], blk_t_scale [ceil(K/128), ceil(M/128)])``."""
    assert x.ndim == 2
    tok, tok_s = _rows(x)
    _, _, qt, st = quant_blocks(x.contiguous(), transposed=True)
    return tok, tok_s, qt[0], st[0]


def fp8cast_blockwise_transpose(x: torch.Tensor) -> Four:
    """``(fp8 [M,K], scale [ceil(M/128), ceil(K/128)], fp8_t [K,M], scale_t [ceil(K/128), ceil(M/128)])``."""
    assert x.ndim == 2
    q, s, qt, st = quant_blocks(x.contiguous(), transposed=True)
    return q[0], s[0], qt[0], st[0]


def fp8cast_blockwise_transpose_batched(x: torch.Tensor) -> Four:
    """The 3-D form: ``x [G,N,K]`` -> payloads ``[G,N,K]`` / ``[G,K,N]`` and scales ``[G,nb,kb]`` / ``[G,kb,nb]``."""
    assert x.ndim == 3
    return quant_blocks(x.contiguous(), transposed=True)
