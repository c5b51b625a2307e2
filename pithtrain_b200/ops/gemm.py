"""bf16 GEMMs on the tcgen05 kernel family (dense, M-grouped, K-grouped) and their fp32 oracles.

Layout vocabulary: an operand is "K-major" when its reduction dimension is contiguous in memory and
"MN-major" when it is strided. The kernel reads either, so the wrappers below never transpose:

* ``gemm_nt(x[M,K], w[N,K])``        forward  ``x @ w.T``        (both K-major)
* ``gemm_nn(dy[M,N], w[N,K])``       dgrad    ``dy @ w``         (B MN-major)
* ``gemm_tn(dy[M,N], x[M,K])``       wgrad    ``dy.T @ x``       (both MN-major)

Grouped variants take ``offs`` (int32 ``[G+1]`` device tensor of row offsets, group sizes multiples
of 16 for the K-grouped form); nothing is read back to the host.
Counterparts in the reference: pithtrain/operators/grouped_linear.py:18-55 (F.grouped_mm) and the
dense ``nn.Linear`` calls.
"""

from __future__ import annotations

import os

import torch

from .. import _native

DENSE, MGROUP, KGROUP = 0, 1, 2

# Module-level switches used by tests and tuning runs.
USE_TMA_STORE = True
FORCE_BN = 0
# accumulate epilogue: 0 = staged coalesced read-modify-write, 1 = per-thread rows, 2 = TMA reduce-add
ACC_EPILOGUE = 2


def _launch(a, b, d, mode, M, N, K, a_mn, b_mn, a_shape, lda, b_shape, ldb, d_rows, ldd,
            offs=None, num_groups=0, b_group_rows=0, d_group_stride=0, accumulate=False,
            max_ctas=0, a_idx=None, a_idx_div=1):
    L = _native.lib()
    out_fp32 = 1 if d.dtype == torch.float32 else 0
    rc = L.pt_gemm_bf16(
        a.data_ptr(), b.data_ptr(), d.data_ptr(), mode, M, N, K, int(a_mn), int(b_mn),
        a_shape[0], a_shape[1], lda, b_shape[0], b_shape[1], ldb, d_rows, ldd,
        None if offs is None else offs.data_ptr(), num_groups, b_group_rows, d_group_stride,
        out_fp32, int(accumulate), int(USE_TMA_STORE), ACC_EPILOGUE, FORCE_BN, max_ctas,
        None if a_idx is None else a_idx.data_ptr(), int(a_idx_div), 0 if a_idx is None else a_idx.numel(),
        _native.stream_ptr(),
    )
    _native.check(rc, "pt_gemm_bf16")


def _native_ok(*ts: torch.Tensor) -> bool:
    ok = all(t.is_cuda and t.dtype == torch.bfloat16 for t in ts)
    if ok:
        _native.lib()
    return ok


def _chk2d(t: torch.Tensor, name: str):
    assert t.dim() == 2 and t.stride(1) == 1, f"{name} must be row-major 2-D, got {t.shape} {t.stride()}"
    assert t.dtype == torch.bfloat16, f"{name} must be bf16"
    assert t.stride(0) % 8 == 0 and t.data_ptr() % 16 == 0, f"{name} must be 16-byte aligned"


# Plain dense NT products (fresh bf16 output, no accumulation) run on the 2-CTA kernel of csrc/gemm_2cta.cu: a CTA pair
# shares each B tile, which measured 6-11 % faster than the single-CTA family at the model's projection shapes.
USE_2CTA = True


def _gemm2cta_nt(x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    M, K = x.shape
    N = w.shape[0]
    out = torch.empty((M, N), dtype=torch.bfloat16, device=x.device)
    rc = _native.lib().pt_gemm2cta_nt(x.data_ptr(), w.data_ptr(), out.data_ptr(), M, N, K, x.stride(0), w.stride(0),
                                      out.stride(0), _native.stream_ptr())
    _native.check(rc, "pt_gemm2cta_nt")
    return out


@torch.no_grad()
def gemm_nt(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor | None = None,
            accumulate: bool = False, out_dtype: torch.dtype | None = None) -> torch.Tensor:
    """``x[M,K] @ w[N,K].T -> [M,N]``."""
    out_dtype = out_dtype or x.dtype
    if (USE_2CTA and out is None and not accumulate and out_dtype == torch.bfloat16 and _native_ok(x, w)
            and x.shape[1] % 8 == 0 and w.shape[0] % 8 == 0):
        _chk2d(x, "x"); _chk2d(w, "w")
        return _gemm2cta_nt(x, w)
    if not _native_ok(x, w):
        r = x.float() @ w.float().t()
        if out is None:
            return r.to(out_dtype)
        out.copy_(out.float() + r if accumulate else r)
        return out
    _chk2d(x, "x"); _chk2d(w, "w")
    M, K = x.shape
    N = w.shape[0]
    assert w.shape[1] == K
    if out is None:
        out = torch.empty((M, N), dtype=out_dtype, device=x.device)
    _launch(x, w, out, DENSE, M, N, K, False, False, (M, K), x.stride(0), (N, K), w.stride(0),
            M, out.stride(0), accumulate=accumulate)
    return out


@torch.no_grad()
def gemm_nn(dy: torch.Tensor, w: torch.Tensor, out: torch.Tensor | None = None,
            accumulate: bool = False, out_dtype: torch.dtype | None = None) -> torch.Tensor:
    """``dy[M,N] @ w[N,K] -> [M,K]`` (reduction over N; ``w`` is read MN-major)."""
    out_dtype = out_dtype or dy.dtype
    if not _native_ok(dy, w):
        r = dy.float() @ w.float()
        if out is None:
            return r.to(out_dtype)
        out.copy_(out.float() + r if accumulate else r)
        return out
    _chk2d(dy, "dy"); _chk2d(w, "w")
    M, N = dy.shape
    K = w.shape[1]
    assert w.shape[0] == N
    if out is None:
        out = torch.empty((M, K), dtype=out_dtype, device=dy.device)
    # GEMM view: D[M, K] = A[M, red=N] * B[red=N, K]
    _launch(dy, w, out, DENSE, M, K, N, False, True, (M, N), dy.stride(0), (N, K), w.stride(0),
            M, out.stride(0), accumulate=accumulate)
    return out


@torch.no_grad()
def gemm_tn(dy: torch.Tensor, x: torch.Tensor, out: torch.Tensor | None = None,
            accumulate: bool = False, out_dtype: torch.dtype | None = None) -> torch.Tensor:
    """``dy[M,N].T @ x[M,K] -> [N,K]`` (reduction over rows; both operands read MN-major)."""
    out_dtype = out_dtype or dy.dtype
    if not _native_ok(dy, x):
        r = dy.float().t() @ x.float()
        if out is None:
            return r.to(out_dtype)
        out.copy_(out.float() + r if accumulate else r)
        return out
    _chk2d(dy, "dy"); _chk2d(x, "x")
    M, N = dy.shape
    K = x.shape[1]
    assert x.shape[0] == M
    if out is None:
        assert not accumulate
        out = torch.empty((N, K), dtype=out_dtype, device=dy.device)
    _launch(dy, x, out, DENSE, N, K, M, True, True, (M, N), dy.stride(0), (M, K), x.stride(0),
            N, out.stride(0), accumulate=accumulate)
    return out


# ------------------------------------------------------------------------------------------------
# grouped
# ------------------------------------------------------------------------------------------------
def _group_loop(offs: torch.Tensor):
    o = offs.tolist()
    return [(g, o[g], o[g + 1]) for g in range(len(o) - 1)]


@torch.no_grad()
def _gathered(x: torch.Tensor, a_idx: torch.Tensor, div: int) -> torch.Tensor:
    """Reference of the in-kernel row gather: ``x[a_idx // div]`` with zero rows for negative indices."""
    ii = a_idx.long()
    rows = x[(ii.clamp(min=0) // div)]
    return torch.where((ii >= 0).unsqueeze(-1), rows, torch.zeros((), dtype=x.dtype, device=x.device))


@torch.no_grad()
def grouped_gemm_nt(x: torch.Tensor, w: torch.Tensor, offs: torch.Tensor, out: torch.Tensor | None = None,
                    a_idx: torch.Tensor | None = None, a_idx_div: int = 1) -> torch.Tensor:
    """Rows ``[offs[g], offs[g+1])`` of ``x[R,K]`` times ``w[g][N,K].T`` -> ``out[R,N]``.

    With ``a_idx`` (int32 ``[R]``) the GEMM's row ``r`` is ``x[a_idx[r] // a_idx_div]`` (zeros for a
    negative index): the expert-order gather happens inside the TMA producer and the gathered copy of
    the activations is never written. Rows at or beyond ``offs[-1]`` are left untouched.
    """
    G, N, K = w.shape
    R = x.shape[0] if a_idx is None else int(a_idx.numel())
    if out is None:
        out = torch.empty((R, N), dtype=x.dtype, device=x.device)
    if not _native_ok(x, w):
        xs = x if a_idx is None else _gathered(x, a_idx, a_idx_div)
        for g, a, b in _group_loop(offs):
            out[a:b] = (xs[a:b].float() @ w[g].float().t()).to(out.dtype)
        return out
    _chk2d(x, "x")
    assert w.is_contiguous() and w.dtype == torch.bfloat16 and offs.dtype == torch.int32
    assert a_idx is None or (a_idx.dtype == torch.int32 and a_idx.is_contiguous())
    _launch(x, w, out, MGROUP, R, N, K, False, False, (x.shape[0], K), x.stride(0), (G * N, K), K,
            R, out.stride(0), offs=offs, num_groups=G, b_group_rows=N, a_idx=a_idx, a_idx_div=a_idx_div)
    return out


@torch.no_grad()
def grouped_gemm_nn(dy: torch.Tensor, w: torch.Tensor, offs: torch.Tensor, out: torch.Tensor | None = None,
                    a_idx: torch.Tensor | None = None, a_idx_div: int = 1) -> torch.Tensor:
    """Rows of group g of ``dy[R,N]`` times ``w[g][N,K]`` -> ``out[R,K]`` (expert dgrad); ``a_idx`` gathers
    the rows of ``dy`` inside the kernel as in :func:`grouped_gemm_nt`."""
    G, N, K = w.shape
    R = dy.shape[0] if a_idx is None else int(a_idx.numel())
    if out is None:
        out = torch.empty((R, K), dtype=dy.dtype, device=dy.device)
    if not _native_ok(dy, w):
        ds = dy if a_idx is None else _gathered(dy, a_idx, a_idx_div)
        for g, a, b in _group_loop(offs):
            out[a:b] = (ds[a:b].float() @ w[g].float()).to(out.dtype)
        return out
    _chk2d(dy, "dy")
    assert w.is_contiguous() and w.dtype == torch.bfloat16 and offs.dtype == torch.int32
    assert N % 64 == 0, "reduction dim of a grouped dgrad must be a multiple of 64"
    _launch(dy, w, out, MGROUP, R, K, N, False, True, (dy.shape[0], N), dy.stride(0), (G * N, K), K,
            R, out.stride(0), offs=offs, num_groups=G, b_group_rows=N, a_idx=a_idx, a_idx_div=a_idx_div)
    return out


@torch.no_grad()
def grouped_gemm_tn(dy: torch.Tensor, x: torch.Tensor, offs: torch.Tensor, out: torch.Tensor,
                    accumulate: bool = True) -> torch.Tensor:
    """``out[g] (+)= dy[rows_g].T @ x[rows_g]`` with ``out[G,N,K]`` (expert wgrad).

    Group sizes must be multiples of 16; pad rows must be zero in ``dy`` (or ``x``).
    """
    G, N, K = out.shape
    if not _native_ok(dy, x):
        for g, a, b in _group_loop(offs):
            r = dy[a:b].float().t() @ x[a:b].float()
            out[g] = (out[g].float() + r if accumulate else r).to(out.dtype)
        return out
    _chk2d(dy, "dy"); _chk2d(x, "x")
    assert out.is_contiguous() and offs.dtype == torch.int32
    if not accumulate:
        out.zero_()
    R = dy.shape[0]
    _launch(dy, x, out, KGROUP, N, K, 0, True, True, (R, N), dy.stride(0), (R, K), x.stride(0),
            N, K, offs=offs, num_groups=G, d_group_stride=N * K, accumulate=True)
    return out


@torch.no_grad()
def grouped_gemm_tn_pair(dy1: torch.Tensor, x1: torch.Tensor, offs1: torch.Tensor, dy2: torch.Tensor, x2: torch.Tensor,
                         offs2: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """``out[g] += dy1[rows1_g].T @ x1[rows1_g] + dy2[rows2_g].T @ x2[rows2_g]``: the expert weight gradients of two
    micro-batches in one launch. The launch is bound by the read-modify-write of ``out`` (the whole ``[G, N, K]``
    gradient buffer), not by its FLOPs, so one pass for two micro-batches nearly halves its cost."""
    G, N, K = out.shape
    if not (_native_ok(dy1, x1) and _native_ok(dy2, x2)) or N % 8 != 0 or K % 8 != 0:
        grouped_gemm_tn(dy1, x1, offs1, out, accumulate=True)
        return grouped_gemm_tn(dy2, x2, offs2, out, accumulate=True)
    for t, n in ((dy1, "dy1"), (x1, "x1"), (dy2, "dy2"), (x2, "x2")):
        _chk2d(t, n)
    assert out.is_contiguous() and offs1.dtype == torch.int32 and offs2.dtype == torch.int32
    assert dy1.stride(0) == dy2.stride(0) and x1.stride(0) == x2.stride(0)
    rc = _native.lib().pt_gemm_bf16_kgroup2(dy1.data_ptr(), x1.data_ptr(), offs1.data_ptr(), dy1.shape[0], dy2.data_ptr(),
                                            x2.data_ptr(), offs2.data_ptr(), dy2.shape[0], out.data_ptr(), N, K, dy1.stride(0),
                                            x1.stride(0), K, N * K, G, int(out.dtype == torch.float32), _native.stream_ptr())
    _native.check(rc, "pt_gemm_bf16_kgroup2")
    return out
