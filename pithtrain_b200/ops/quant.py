"""FP8 (e4m3) quantisation with power-of-two scales, and the block-scaled FP8 GEMM wrappers.

Recipe per group (1x128 row segment, or 128x128 weight tile): ``a = max(amax, 1e-4)``,
``scale = 2^ceil(log2(a / 448))`` (at least ``2^-126``), ``q = e4m3(x / scale)``. Same numbers as
pithtrain/operators/deepgemm_quantize.py:36-83 of the reference; ``*_ref`` below restate it with
plain tensor ops and are the bit-exact oracles for the CUDA kernels in ``csrc/quant.cu``.

Row scales are stored k-block-major (``[ceil(K/128), ld]``): the layout the GEMM's epilogue reads
coalesced. ``ld`` is the row capacity rounded up to 4.
"""

from __future__ import annotations

from typing import Optional, Tuple

import torch

from .. import _native
from .common import use_native

FP8 = torch.float8_e4m3fn
BLOCK = 128


def _sp():
    return _native.stream_ptr()


def pow2_scale_ref(amax: torch.Tensor) -> torch.Tensor:
    """``2^ceil(log2(max(amax,1e-4)/448))`` computed on the bit pattern, like the kernel."""
    s_in = torch.clamp(amax.float(), min=1e-4) * (1.0 / 448.0)
    bits = s_in.view(torch.int32)
    e = (bits >> 23) + ((bits & 0x7FFFFF) != 0).int()
    e = e.clamp(1, 254)
    return (e << 23).view(torch.float32)


def quant_rows_ref(x: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """``x [R, K]`` -> ``(q [R, K] e4m3, scales [ceil(K/128), R] fp32)``."""
    R, K = x.shape
    kb = (K + BLOCK - 1) // BLOCK
    xp = torch.zeros((R, kb * BLOCK), dtype=torch.float32, device=x.device)
    xp[:, :K] = x.float()
    g = xp.view(R, kb, BLOCK)
    scale = pow2_scale_ref(g.abs().amax(-1))  # [R, kb]
    q = (g / scale.unsqueeze(-1)).view(R, kb * BLOCK)[:, :K].to(FP8)
    return q, scale.t().contiguous()


def quant_blocks_ref(w: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """``w [G, N, K]`` -> ``(q [G, N, K] e4m3, scales [G, ceil(N/128), ceil(K/128)])``."""
    G, N, K = w.shape
    nb, kb = (N + BLOCK - 1) // BLOCK, (K + BLOCK - 1) // BLOCK
    wp = torch.zeros((G, nb * BLOCK, kb * BLOCK), dtype=torch.float32, device=w.device)
    wp[:, :N, :K] = w.float()
    t = wp.view(G, nb, BLOCK, kb, BLOCK)
    scale = pow2_scale_ref(t.abs().amax(dim=(2, 4)))  # [G, nb, kb]
    q = (t / scale[:, :, None, :, None]).view(G, nb * BLOCK, kb * BLOCK)[:, :N, :K].to(FP8)
    return q.contiguous(), scale


def dequant_rows(q: torch.Tensor, s: torch.Tensor) -> torch.Tensor:
    R, K = q.shape
    sc = s[:, :R].t().repeat_interleave(BLOCK, dim=1)[:, :K]
    return q.float() * sc


def dequant_blocks(q: torch.Tensor, s: torch.Tensor) -> torch.Tensor:
    G, N, K = q.shape
    sc = s.repeat_interleave(BLOCK, dim=1).repeat_interleave(BLOCK, dim=2)[:, :N, :K]
    return q.float() * sc


def quant_rows(x: torch.Tensor, idx: Optional[torch.Tensor] = None, div: int = 1,
               n_rows: Optional[torch.Tensor] = None, rows: Optional[int] = None) -> Tuple[torch.Tensor, torch.Tensor]:
    """Row-wise 1x128 quantisation of ``x [*, K]`` (bf16), optionally gathering ``x[idx // div]``.

    Returns ``(q [R, K], scales [ceil(K/128), ld])`` with ``R = len(idx)`` or ``rows`` or ``x.shape[0]``.
    Rows at or past the device-side count ``n_rows`` are left unwritten.
    """
    K = x.shape[-1]
    R = int(idx.numel()) if idx is not None else (rows if rows is not None else x.shape[0])
    kb = (K + BLOCK - 1) // BLOCK
    ld = (R + 3) // 4 * 4
    if use_native(x) and x.dtype == torch.bfloat16 and K % 8 == 0 and x.stride(-1) == 1:
        q = torch.empty((R, K), dtype=FP8, device=x.device)
        s = torch.empty((kb, ld), dtype=torch.float32, device=x.device)
        rc = _native.lib().pt_quant_rows(x.data_ptr(), x.stride(0), None if idx is None else idx.data_ptr(), int(div),
                                         None if n_rows is None else n_rows.data_ptr(), R, K, q.data_ptr(),
                                         s.data_ptr(), ld, _sp())
        _native.check(rc, "pt_quant_rows")
        return q, s
    src = x
    if idx is not None:
        ii = idx.long()
        src = torch.where((ii >= 0).unsqueeze(-1), x[(ii.clamp(min=0) // div)], torch.zeros((), dtype=x.dtype, device=x.device))
    q, s = quant_rows_ref(src[:R])
    if ld != R:
        s = torch.cat([s, s.new_zeros(kb, ld - R)], dim=1)
    return q, s


def quant_blocks(w: torch.Tensor, transposed: bool = True):
    """128x128-tile quantisation of ``w [G, N, K]`` (or ``[N, K]``), optionally also of ``w^T``.

    Returns ``(q, s, qT, sT)``; the last two are ``None`` without ``transposed``.
    """
    w3 = w if w.dim() == 3 else w.unsqueeze(0)
    G, N, K = w3.shape
    nb, kb = (N + BLOCK - 1) // BLOCK, (K + BLOCK - 1) // BLOCK
    if use_native(w3) and w3.dtype == torch.bfloat16 and w3.is_contiguous():
        q = torch.empty((G, N, K), dtype=FP8, device=w.device)
        s = torch.empty((G, nb, kb), dtype=torch.float32, device=w.device)
        qt = torch.empty((G, K, N), dtype=FP8, device=w.device) if transposed else None
        st = torch.empty((G, kb, nb), dtype=torch.float32, device=w.device) if transposed else None
        rc = _native.lib().pt_quant_blocks(w3.data_ptr(), G, N, K, q.data_ptr(), None if qt is None else qt.data_ptr(),
                                           s.data_ptr(), None if st is None else st.data_ptr(), _sp())
        _native.check(rc, "pt_quant_blocks")
    else:
        q, s = quant_blocks_ref(w3)
        qt = q.transpose(1, 2).contiguous() if transposed else None
        st = s.transpose(1, 2).contiguous() if transposed else None
    return q, s, qt, st


@torch.no_grad()
def gemm_fp8_nt(a_q: torch.Tensor, a_s: torch.Tensor, b_q: torch.Tensor, b_s: torch.Tensor,
                offs: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None,
                use_tma_store: bool = True) -> torch.Tensor:
    """``out [R, N] (bf16) = dequant(a) @ dequant(b)^T``.

    Dense: ``b_q [N, K]`` (or ``[1, N, K]``), ``b_s [1, nb, kb]``. Grouped: ``b_q [G, N, K]`` and
    ``offs [G+1]`` (int32, device) cut the rows of ``a`` into groups.
    """
    R, K = a_q.shape
    b3 = b_q if b_q.dim() == 3 else b_q.unsqueeze(0)
    G, N, _ = b3.shape
    if out is None:
        out = torch.empty((R, N), dtype=torch.bfloat16, device=a_q.device)
    if a_q.is_cuda:
        if K % 16 != 0 or N % 8 != 0:
            raise ValueError(f"fp8 GEMM needs K % 16 == 0 and N % 8 == 0, got K={K}, N={N}")
        grouped = offs is not None
        rc = _native.lib().pt_gemm_fp8(a_q.data_ptr(), b3.data_ptr(), out.data_ptr(), 1 if grouped else 0, R, N, K,
                                       R, G * N, R, out.stride(0), a_s.data_ptr(), a_s.stride(0), b_s.data_ptr(),
                                       None if offs is None else offs.data_ptr(), G if grouped else 1, N,
                                       int(use_tma_store), 0, _sp())
        _native.check(rc, "pt_gemm_fp8")
        return out
    a = dequant_rows(a_q, a_s)
    b = dequant_blocks(b3, b_s)
    if offs is None:
        out.copy_((a @ b[0].t()).to(out.dtype))
    else:
        o = offs.tolist()
        out.zero_()
        for g in range(G):
            if o[g + 1] > o[g]:
                out[o[g]:o[g + 1]] = (a[o[g]:o[g + 1]] @ b[g].t()).to(out.dtype)
    return out
