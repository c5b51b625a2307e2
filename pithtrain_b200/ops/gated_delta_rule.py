"""Gated delta rule linear attention (Gated DeltaNet), chunked, in plain PyTorch autograd.

Per head the recurrence over a ``[dk, dv]`` state is
``S <- exp(g_t) * S``, ``S <- S + k_t (beta_t (v_t - S^T k_t))^T``, ``o_t = S^T q_t / sqrt(dk)``.
``gated_delta_rule`` evaluates it chunk by chunk (chunk 64): inside a chunk the sequential
dependence is resolved with a triangular solve, across chunks the state is carried — the same
blocking as the library kernel the reference wraps (pithtrain/operators/gated_delta_rule.py:21-56).
``gated_delta_rule_recurrent`` is the token-by-token oracle.
"""

from __future__ import annotations

import torch


def gated_delta_rule_recurrent(q, k, v, g, beta):
    """q,k [B,S,H,dk]; v [B,S,H,dv]; g, beta [B,S,H]. Returns [B,S,H,dv]."""
    B, S, H, dk = q.shape
    dv = v.shape[-1]
    qf, kf, vf = q.float() * dk ** -0.5, k.float(), v.float()
    gf, bf = g.float(), beta.float()
    state = torch.zeros(B, H, dk, dv, dtype=torch.float32, device=q.device)
    outs = []
    for t in range(S):
        state = state * gf[:, t].exp()[..., None, None]
        kt = kf[:, t]
        v_new = (vf[:, t] - torch.einsum("bhkv,bhk->bhv", state, kt)) * bf[:, t][..., None]
        state = state + kt[..., None] * v_new[..., None, :]
        outs.append(torch.einsum("bhkv,bhk->bhv", state, qf[:, t]))
    return torch.stack(outs, dim=1).to(v.dtype)


def gated_delta_rule(q, k, v, g, beta, chunk_size: int = 64):
    """Chunked evaluation; same signature and result as :func:`gated_delta_rule_recurrent`."""
    B, S, H, dk = q.shape
    dv = v.shape[-1]
    C = chunk_size
    pad = (C - S % C) % C
    qf = (q.float() * dk ** -0.5).permute(0, 2, 1, 3)
    kf, vf = k.float().permute(0, 2, 1, 3), v.float().permute(0, 2, 1, 3)
    gf, bf = g.float().permute(0, 2, 1), beta.float().permute(0, 2, 1)
    if pad:
        P = torch.nn.functional.pad
        qf, kf, vf = P(qf, (0, 0, 0, pad)), P(kf, (0, 0, 0, pad)), P(vf, (0, 0, 0, pad))
        gf, bf = P(gf, (0, pad)), P(bf, (0, pad))
    N = (S + pad) // C
    qf, kf, vf = (x.reshape(B, H, N, C, -1) for x in (qf, kf, vf))
    gf, bf = gf.reshape(B, H, N, C), bf.reshape(B, H, N, C)
    gc = gf.cumsum(-1)  # log decay from chunk start to position i (inclusive)
    kb, vb = kf * bf[..., None], vf * bf[..., None]
    # decay between positions j < i inside a chunk
    diff = gc[..., :, None] - gc[..., None, :]
    tril_strict = torch.tril(torch.ones(C, C, dtype=torch.bool, device=q.device), -1)
    tril_incl = torch.tril(torch.ones(C, C, dtype=torch.bool, device=q.device), 0)
    decay = torch.where(tril_incl, diff, torch.full_like(diff, float("-inf"))).exp()
    # (I + A) u = rhs with A strictly lower: A_ij = beta_i <k_i,k_j> decay_ij
    A = (kb @ kf.transpose(-1, -2)) * decay
    A = A.masked_fill(~tril_strict, 0.0)
    eye = torch.eye(C, device=q.device, dtype=torch.float32)
    T = torch.linalg.solve_triangular(eye + A, eye.expand_as(A).contiguous(), upper=False)
    u = T @ vb  # value part of the per-position updates
    w = T @ (kb * gc.exp()[..., None])  # state-dependent part
    state = torch.zeros(B, H, dk, dv, dtype=torch.float32, device=q.device)
    outs = []
    qk = (qf @ kf.transpose(-1, -2)) * decay
    qk = qk.masked_fill(~tril_incl, 0.0)
    for n in range(N):
        v_new = u[:, :, n] - w[:, :, n] @ state  # [B,H,C,dv]
        o_inter = (qf[:, :, n] * gc[:, :, n].exp()[..., None]) @ state
        outs.append(o_inter + qk[:, :, n] @ v_new)
        g_last = gc[:, :, n, -1]
        k_dec = kf[:, :, n] * (g_last[..., None] - gc[:, :, n]).exp()[..., None]
        state = state * g_last.exp()[..., None, None] + k_dec.transpose(-1, -2) @ v_new
    o = torch.stack(outs, dim=2).reshape(B, H, N * C, dv)[:, :, :S]
    return o.permute(0, 2, 1, 3).to(v.dtype)
