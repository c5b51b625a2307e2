"""Gated delta rule linear attention (Gated DeltaNet), chunked, in plain PyTorch autograd.

Per head the recurrence over a ``[dk, dv]`` state is
``S <- exp(g_t) * S``, ``S <- S + k_t (beta_t (v_t - S^T k_t))^T``, ``o_t = S^T q_t / sqrt(dk)``.
``gated_delta_rule`` evaluates it chunk by chunk (chunk 64): inside a chunk the sequential
dependence is resolved with a triangular solve (batched tensor ops over all chunks at once), across
chunks the state is carried by the recurrence kernels of ``csrc/gdr.cu`` (forward and backward, state
resident in shared memory) — the same blocking as the library kernel the reference wraps
(pithtrain/operators/gated_delta_rule.py:21-56).
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


def _chunk_state_math(w, u, qg, kd, a):
    """The pass over the chunks in tensor ops (CPU path and oracle of the kernel): returns ``v_new, o_inter``.
    ``w, qg, kd [B,H,N,C,dk]``, ``u [B,H,N,C,dv]``, ``a [B,H,N]``."""
    B, H, N, C, dk = w.shape
    state = torch.zeros(B, H, dk, u.shape[-1], dtype=torch.float32, device=w.device)
    v_out, o_out = [], []
    for n in range(N):
        v_new = u[:, :, n] - w[:, :, n] @ state
        o_out.append(qg[:, :, n] @ state)
        v_out.append(v_new)
        state = state * a[:, :, n, None, None] + kd[:, :, n].transpose(-1, -2) @ v_new
    return torch.stack(v_out, dim=2), torch.stack(o_out, dim=2)


class _ChunkState(torch.autograd.Function):
    """The sequential pass over the chunks on the recurrence kernels of ``csrc/gdr.cu`` (state resident in shared
    memory, one CTA per head and 32-column value slice), forward and backward."""

    @staticmethod
    def forward(ctx, w, u, qg, kd, a):
        from .. import _native

        B, H, N, C, dk = w.shape
        dv = u.shape[-1]
        w, u, qg, kd, a = (t.contiguous() for t in (w, u, qg, kd, a))
        v_new, o_inter = torch.empty_like(u), torch.empty_like(u)
        states = torch.empty(B, H, N, dk, dv, dtype=torch.float32, device=w.device)
        rc = _native.lib().pt_gdr_state_fwd(w.data_ptr(), u.data_ptr(), qg.data_ptr(), kd.data_ptr(), a.data_ptr(),
                                            v_new.data_ptr(), o_inter.data_ptr(), states.data_ptr(), B * H, N, dk, dv,
                                            _native.stream_ptr())
        _native.check(rc, "pt_gdr_state_fwd")
        ctx.save_for_backward(w, qg, kd, a, v_new, states)
        return v_new, o_inter

    @staticmethod
    def backward(ctx, d_vnew, d_o):
        from .. import _native

        w, qg, kd, a, v_new, states = ctx.saved_tensors
        B, H, N, C, dk = w.shape
        dv = v_new.shape[-1]
        d_vnew = torch.zeros_like(v_new) if d_vnew is None else d_vnew.contiguous()
        d_o = torch.zeros_like(v_new) if d_o is None else d_o.contiguous()
        d_u = torch.empty_like(v_new)
        d_w, d_qg, d_kd = torch.zeros_like(w), torch.zeros_like(w), torch.zeros_like(w)
        d_a = torch.zeros_like(a)
        rc = _native.lib().pt_gdr_state_bwd(w.data_ptr(), qg.data_ptr(), kd.data_ptr(), a.data_ptr(), v_new.data_ptr(),
                                            states.data_ptr(), d_o.data_ptr(), d_vnew.data_ptr(), d_u.data_ptr(),
                                            d_w.data_ptr(), d_qg.data_ptr(), d_kd.data_ptr(), d_a.data_ptr(), B * H, N, dk, dv,
                                            _native.stream_ptr())
        _native.check(rc, "pt_gdr_state_bwd")
        return d_w, d_u, d_qg, d_kd, d_a


def chunk_state(w, u, qg, kd, a):
    """``v_new, o_inter`` of the pass over the chunks: the kernel on GPUs (fp32, chunk 64, dk 64 or 128, dv a multiple
    of 32), the tensor-op loop otherwise."""
    if w.is_cuda and w.shape[3] == 64 and w.shape[4] in (64, 128) and u.shape[-1] % 32 == 0:
        return _ChunkState.apply(w, u, qg, kd, a)
    return _chunk_state_math(w, u, qg, kd, a)


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
    qk = (qf @ kf.transpose(-1, -2)) * decay
    qk = qk.masked_fill(~tril_incl, 0.0)
    # the sequential part: v_new_n = u_n - w_n S_n, o_inter_n = (q_n e^{gc}) S_n, S_{n+1} = e^{g_last} S_n + kd_n^T v_new_n
    g_last = gc[..., -1]
    qg = qf * gc.exp()[..., None]
    kd = kf * (g_last[..., None] - gc).exp()[..., None]
    v_new, o_inter = chunk_state(w, u, qg, kd, g_last.exp())
    outs = o_inter + qk @ v_new
    o = outs.reshape(B, H, N * C, dv)[:, :, :S]
    return o.permute(0, 2, 1, 3).to(v.dtype)
