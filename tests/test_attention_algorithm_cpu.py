"""The arithmetic of ``csrc/attention.cu`` restated tile by tile in PyTorch: scores in the log2 domain, one running
reference maximum per row that is only raised (and O rescaled) when a tile's maximum exceeds it by more than 2^8,
P rounded to bf16 before the PV product, fp32 accumulation, final division by the row sum and
``lse = m_ref * ln 2 + ln l``. The restatement must agree with plain softmax attention; it pins down the algorithm
the kernel implements independently of its PTX."""
import math

import pytest
import torch

from pithtrain_b200.ops.attention import attention_ref

TILE = 128
RESCALE_LOG2 = 8.0


def tiled_lazy_attention(q, k, v, scale):
    """q [S, D], k/v [S, D] of one head, causal; returns (out [S, D] bf16, lse [S] fp32, number of rescales)."""
    S, D = q.shape
    scale_log2 = scale * math.log2(math.e)
    out = torch.empty(S, D, dtype=torch.bfloat16)
    lse = torch.empty(S)
    rescales = 0
    for q0 in range(0, S, TILE):
        qt = q[q0:q0 + TILE].float()
        rows = torch.arange(q0, q0 + TILE).unsqueeze(1)
        m_ref = torch.full((TILE,), -math.inf)
        l = torch.zeros(TILE)
        O = torch.zeros(TILE, D)
        for j in range(q0 // TILE + 1):
            kt, vt = k[j * TILE:(j + 1) * TILE].float(), v[j * TILE:(j + 1) * TILE].float()
            s = qt @ kt.t()  # fp32 accumulator of the QK^T MMA
            if j == q0 // TILE:
                cols = torch.arange(j * TILE, (j + 1) * TILE).unsqueeze(0)
                s = s.masked_fill(cols > rows, -math.inf)
            m_new = torch.maximum(m_ref, s.max(dim=1).values * scale_log2)
            if j == 0:
                m_ref = m_new
            else:
                grow = m_new > m_ref + RESCALE_LOG2
                # the kernel decides per warp (32 rows): if any row of the warp grows, all rows of the warp rescale
                warp_any = grow.view(-1, 32).any(dim=1).repeat_interleave(32)
                alpha = torch.where(warp_any, torch.exp2(m_ref - m_new), torch.ones_like(m_ref))
                m_ref = torch.where(warp_any, m_new, m_ref)
                l = l * alpha
                O = O * alpha.unsqueeze(1)
                rescales += int(warp_any.view(-1, 32)[:, 0].sum())
            p = torch.exp2(s * scale_log2 - m_ref.unsqueeze(1))  # masked entries: exp2(-inf) = 0
            l = l + p.sum(dim=1)
            O = O + p.bfloat16().float() @ vt  # P is stored as bf16 for the PV MMA
        out[q0:q0 + TILE] = (O / l.unsqueeze(1)).bfloat16()
        lse[q0:q0 + TILE] = m_ref * math.log(2.0) + torch.log(l)
    return out, lse, rescales


@pytest.mark.parametrize("S,spread", [(256, 1.0), (512, 4.0), (384, 12.0)])
def test_tiled_lazy_rescale_attention_matches_softmax_attention(S, spread):
    torch.manual_seed(0)
    D = 128
    q = (torch.randn(S, D) * spread).bfloat16()
    k = torch.randn(S, D).bfloat16()
    v = torch.randn(S, D).bfloat16()
    scale = D ** -0.5
    out, lse, rescales = tiled_lazy_attention(q, k, v, scale)
    ref, ref_lse = attention_ref(q.view(1, S, 1, D), k.view(1, S, 1, D), v.view(1, S, 1, D), causal=True, scale=scale,
                                 return_lse=True)
    ref, ref_lse = ref.view(S, D).float(), ref_lse.view(S)
    assert torch.allclose(lse, ref_lse, atol=2e-3, rtol=1e-4)
    err = (out.float() - ref).abs().max()
    assert float(err) < 3e-2, float(err)  # bf16 rounding of P and of the output
    if spread >= 12.0:
        assert rescales > 0  # large score spreads do exercise the rescale branch
    if spread <= 1.0:
        assert rescales == 0  # and ordinary ones never leave the first reference maximum by more than 2^8


def test_stale_reference_maximum_stays_exact():
    """A row whose later tiles are up to 2^8 larger than its reference maximum keeps that reference: p exceeds 1 but the
    ratio O / l is unchanged, so the result equals the eagerly rescaled one."""
    torch.manual_seed(1)
    S, D = 256, 128
    q, k, v = torch.randn(S, D).bfloat16(), torch.randn(S, D).bfloat16(), torch.randn(S, D).bfloat16()
    with torch.no_grad():
        k[200] = q[255] * 0.35  # a late key that raises row 255's maximum by a few units, below the threshold
    out, lse, rescales = tiled_lazy_attention(q, k, v, D ** -0.5)
    ref, ref_lse = attention_ref(q.view(1, S, 1, D), k.view(1, S, 1, D), v.view(1, S, 1, D), causal=True, scale=D ** -0.5,
                                 return_lse=True)
    assert rescales == 0
    assert torch.allclose(lse, ref_lse.view(S), atol=2e-3) and float((out.float() - ref.view(S, D).float()).abs().max()) < 3e-2
