"""Muon and AdamW over owner-sharded parameters.

Muon: SGD momentum, Nesterov blend, quintic Newton-Schulz orthogonalisation (5 steps, bf16,
batched over stacked experts), Moonlight scale ``0.2*sqrt(max(n,m))``, decoupled weight decay —
the update rule of pithtrain/modules/optimizer.py:34-63,155-211. Because a parameter's owner holds
the whole matrix and its fully reduced gradient (see :mod:`pithtrain_b200.parallel.flat_shard`),
Newton-Schulz runs locally on ~1/G of the weights per rank and the regular parameter all-gather
publishes the result; the reference's gather-per-weight and owner broadcasts have no counterpart.

Implementation notes. Work is done on contiguous *units*: a plain parameter, or the fused
``[E, 2, I, H]`` storage behind an expert gate/up pair (each ``[I, H]`` matrix is still
orthogonalised on its own). On CUDA the momentum update and the final ``w = w*(1-lr*wd) - lr*s*O``
are single kernels over the unit; the matmuls of the iteration go to batched GEMMs. The momentum
buffers can live in pinned host memory (``offload_state``): chunks are prefetched on a copy
stream while the previous chunk is being orthogonalised and written back on another, which is what
lets a 30B-parameter model train on one 180 GB GPU.

Both optimizers read ``p.main_grad`` when present (flat accumulators, possibly a different dtype
than the parameter) and ``p.grad`` otherwise, and skip parameters this rank does not own.
"""

from __future__ import annotations

from typing import Dict, List, Optional

import torch

from .. import _native


def _grad_of(p: torch.Tensor) -> Optional[torch.Tensor]:
    g = getattr(p, "main_grad", None)
    return g if g is not None else p.grad


def _grad_scale_of(p: torch.Tensor) -> Optional[torch.Tensor]:
    """Pending factor on ``p``'s accumulated gradient (a device scalar kept by its flat shard group)."""
    grp = getattr(p, "_shard_group", None)
    return getattr(grp, "grad_scale", None) if grp is not None else None


def _owned(p: torch.Tensor) -> bool:
    grp = getattr(p, "_shard_group", None)
    return True if grp is None else grp.is_owned(p)


def zeropower_via_newtonschulz5(Gm: torch.Tensor, steps: int = 5) -> torch.Tensor:
    """Quintic Newton-Schulz iteration towards the orthogonal polar factor, batched over leading dims.

    The iteration is ``X <- aX + (bA + cA^2)X`` with ``A = X X^T`` on the wide orientation of
    ``X0 = G / (|G|_F + 1e-7)``, in bf16 (pithtrain/modules/optimizer.py:34-57 of the reference). It is
    evaluated so that the large ``[m, n]`` operand is only ever touched by matrix products:

    * ``aX + BX = (B + aI) X`` — the ``a`` goes onto the diagonal of the small ``[m, m]`` matrix, so no
      copy of ``X`` is made for a ``beta`` term;
    * the Frobenius normalisation is folded into the first step: ``A = s^2 G G^T`` and
      ``X1 = (s (B + aI)) G`` with ``s = 1/(|G|_F + 1e-7)`` — ``G`` itself is never rescaled;
    * a tall input is used through its transposed view and the last product is formed directly in the
      input's orientation (``X^T (B + aI)``, the small factor being symmetric), so the result needs no
      transposing copy.
    """
    assert Gm.ndim >= 2
    if _own_gemm_usable(Gm):
        return newtonschulz5_own_gemm(Gm, steps)
    a, b, c = 3.4445, -4.7750, 2.0315
    G = Gm.to(torch.bfloat16)
    squeeze = G.ndim == 2
    if squeeze:
        G = G.unsqueeze(0)
    lead = G.shape[:-2]
    G = G.reshape(-1, G.shape[-2], G.shape[-1])
    tall = G.size(-2) > G.size(-1)
    X = G.mT if tall else G  # wide orientation [m, n], m <= n (a view)
    if steps <= 0:
        nrm = torch.linalg.vector_norm(G, dim=(-2, -1), keepdim=True, dtype=torch.float32)
        out = G / (nrm + 1e-7).to(G.dtype)
    else:
        nrm = torch.linalg.vector_norm(G, dim=(-2, -1), keepdim=True, dtype=torch.float32)
        s = 1.0 / (nrm + 1e-7)
        s1, s2 = s.to(G.dtype), (s * s).to(G.dtype)
        out = None
        for it in range(steps):
            A = torch.bmm(X, X.mT)
            if it == 0:
                A.mul_(s2)
            B = torch.baddbmm(A, A, A, beta=b, alpha=c)
            B.diagonal(dim1=-2, dim2=-1).add_(a)
            if it == 0:
                B.mul_(s1)
            last = it == steps - 1
            if last and tall:
                out = torch.bmm(X.mT, B)  # [n, m]: the input's own orientation
            else:
                X = torch.bmm(B, X)
                if last:
                    out = X
    out = out.reshape(*lead, out.shape[-2], out.shape[-1])
    return out.squeeze(0) if squeeze else out


def newtonschulz5_own_gemm(Gm: torch.Tensor, steps: int = 5) -> torch.Tensor:
    """The same iteration on this package's own tcgen05 GEMM family instead of the library's batched products.

    A stack ``[E, r, c]`` is one row-grouped problem: ``Y Y^T`` (wide) is an M-grouped NT product of the rows of every
    matrix against itself, ``Y^T Y`` (tall) a K-grouped TN product, ``A A`` an M-grouped NT product (``A`` is
    symmetric), and the update ``(B + aI) Y`` / ``Y (B + aI)`` an M-grouped NN product — the operand layouts of the
    forward, input-gradient and weight-gradient GEMMs of a grouped linear layer. ``Y`` stays in the input's
    orientation throughout, so neither case needs a transposed copy. Selected for CUDA inputs by
    ``PITHTRAIN_NS_GEMM=own``; not the default until it has been timed against the batched library products.
    """
    from ..ops import gemm as G_

    a, b, c = 3.4445, -4.7750, 2.0315
    G = Gm.to(torch.bfloat16)
    lead = G.shape[:-2]
    G = G.reshape(-1, G.shape[-2], G.shape[-1]).contiguous()
    E, r, cdim = G.shape
    wide = r <= cdim
    m = r if wide else cdim
    dev = G.device
    nrm = torch.linalg.vector_norm(G, dim=(-2, -1), keepdim=True, dtype=torch.float32)
    s = 1.0 / (nrm + 1e-7)
    s1, s2 = s.to(G.dtype), (s * s).to(G.dtype)
    offs_r = (torch.arange(E + 1, device=dev, dtype=torch.int32) * r)
    offs_m = (torch.arange(E + 1, device=dev, dtype=torch.int32) * m)
    Y = G.view(E * r, cdim)
    eye_a = None
    for it in range(max(steps, 0)):
        Y3 = Y.view(E, r, cdim)
        if wide:
            A = G_.grouped_gemm_nt(Y, Y3, offs_r).view(E, m, m)
        else:
            A = G_.grouped_gemm_tn(Y, Y, offs_r, torch.zeros((E, m, m), dtype=G.dtype, device=dev), accumulate=True)
        if it == 0:
            A = A * s2
        A2 = A.reshape(E * m, m)
        AA = G_.grouped_gemm_nt(A2, A.contiguous(), offs_m).view(E, m, m)
        B = b * A + c * AA
        B.diagonal(dim1=-2, dim2=-1).add_(a)
        if it == 0:
            B = B * s1
        B = B.contiguous()
        if wide:
            Y = G_.grouped_gemm_nn(B.view(E * m, m), Y3, offs_m)  # (B + aI) Y
        else:
            Y = G_.grouped_gemm_nn(Y, B, offs_r)  # Y (B + aI)
    if steps <= 0:
        Y = (G * s1).view(E * r, cdim)
    return Y.view(*lead, r, cdim)


def _own_gemm_usable(G: torch.Tensor) -> bool:
    import os

    if os.environ.get("PITHTRAIN_NS_GEMM", "library") != "own" or not G.is_cuda:
        return False
    r, c = G.shape[-2], G.shape[-1]
    return min(r, c) % 64 == 0 and r % 16 == 0 and c % 8 == 0


def muon_scale_factor(n: int, m: int) -> float:
    return 0.2 * max(n, m) ** 0.5


def orthogonalized_updates(params: List[torch.Tensor], updates: List[torch.Tensor], steps: int = 5) -> List[torch.Tensor]:
    """Orthogonalise and scale each update; every entry is a full matrix (or a stack of them)."""
    out = []
    for p, u in zip(params, updates):
        o = zeropower_via_newtonschulz5(u, steps=steps).to(p.dtype)
        out.append(o * muon_scale_factor(u.size(-2), u.size(-1)))
    return out


class _Unit:
    """Contiguous storage that Muon processes in one go."""

    __slots__ = ("w", "g", "params", "key", "gscale")

    def __init__(self, w, g, params, key):
        self.w, self.g, self.params, self.key = w, g, params, key
        self.gscale = _grad_scale_of(params[0])


class Muon(torch.optim.Optimizer):
    """Muon for 2-D hidden weights and stacked 3-D expert weights; pass only Muon-eligible parameters."""

    def __init__(self, params, lr: float = 0.02, momentum: float = 0.95, weight_decay: float = 0.1,
                 momentum_dtype: torch.dtype = torch.float32, offload_state: bool = False,
                 max_chunk_elems: int = 1 << 28, device_state_budget: int = 0):
        defaults = dict(lr=lr, momentum=momentum, weight_decay=weight_decay)
        super().__init__(params, defaults)
        self.momentum_dtype = momentum_dtype
        self.offload_state = offload_state
        # with offload_state: bytes of momentum that may stay on the device anyway (largest use of spare HBM:
        # every byte kept resident is a byte that does not cross PCIe twice per step)
        self.device_state_budget = int(device_state_budget)
        self._device_state_bytes = 0
        self.max_chunk_elems = max_chunk_elems
        self._unit_state: Dict[int, torch.Tensor] = {}
        self._streams = None
        self._stage: List[torch.Tensor] = []

    # ------------------------------------------------------------------ state
    def _new_state(self, like: torch.Tensor) -> torch.Tensor:
        if self.offload_state and like.is_cuda:
            nbytes = like.numel() * torch.empty((), dtype=self.momentum_dtype).element_size()
            if self._device_state_bytes + nbytes > self.device_state_budget:
                return torch.zeros(like.shape, dtype=self.momentum_dtype, device="cpu", pin_memory=True)
            self._device_state_bytes += nbytes
        return torch.zeros(like.shape, dtype=self.momentum_dtype, device=like.device)

    def _units(self, group) -> List[_Unit]:
        """Contiguous units of this rank's owned parameters; creates momentum state on first use."""
        units, seen = [], set()
        for p in group["params"]:
            g = _grad_of(p)
            if g is None or not _owned(p):
                continue
            fusion = getattr(p, "_fusion", None)
            fw = fusion[0] if fusion is not None else None
            if fw is not None and fw.layout == "pair" and fw.weight() is not None and fw.fused_grad is not None \
                    and getattr(p, "main_grad", None) is not None:
                if id(fw) in seen:
                    continue
                seen.add(id(fw))
                E, two, I, H = fw.fused.shape
                w = fw.fused.view(E * 2, I, H)
                gg = fw.fused_grad.view(E * 2, I, H)
                key = id(fw)
                if key not in self._unit_state:
                    st = self._new_state(w)
                    self._unit_state[key] = st
                    sv = st.view(E, 2, I, H)
                    for i, q in enumerate(fw.params):
                        prev = self.state[q].get("momentum_buffer")
                        if prev is not None:  # restored from a checkpoint before the first step
                            sv[:, i].copy_(prev)
                        self.state[q]["momentum_buffer"] = sv[:, i]
                units.append(_Unit(w, gg, list(fw.params), key))
            else:
                key = id(p)
                if key not in self._unit_state:
                    if "momentum_buffer" in self.state[p]:  # restored from a checkpoint
                        prev = self.state[p]["momentum_buffer"]
                        st = self._new_state(p)
                        st.copy_(prev)
                        self._unit_state[key] = st
                        self.state[p]["momentum_buffer"] = st
                    else:
                        self._unit_state[key] = self._new_state(p)
                        self.state[p]["momentum_buffer"] = self._unit_state[key]
                w, gg = (p.data, g) if p.ndim >= 3 else (p.data.unsqueeze(0), g.unsqueeze(0))
                units.append(_Unit(w, gg, [p], key))
        return units

    # ------------------------------------------------------------------ step
    @torch.no_grad()
    def step(self, closure=None):
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        for group in self.param_groups:
            beta, lr, wd = group["momentum"], group["lr"], group["weight_decay"]
            work = []
            for u in self._units(group):
                st = self._unit_state[u.key]
                st3 = st if st.ndim >= 3 else st.unsqueeze(0)
                per = u.w[0].numel()
                chunk = max(1, self.max_chunk_elems // per)
                for s in range(0, u.w.shape[0], chunk):
                    sl = slice(s, min(s + chunk, u.w.shape[0]))
                    work.append((u.w[sl], u.g[sl], st3[sl], u.gscale))
            if not work:
                continue
            if self.offload_state and work[0][0].is_cuda:
                host = [item for item in work if not item[2].is_cuda]
                resident = [item for item in work if item[2].is_cuda]
                # host-resident chunks first, so their write-back drains while the resident ones compute
                if host:
                    self._run_offloaded(host, beta, lr, wd, tail=resident)
                else:
                    for w, g, st, gs in resident:
                        self._update_chunk(w, g, st, beta, lr, wd, gs)
            else:
                for w, g, st, gs in work:
                    self._update_chunk(w, g, st, beta, lr, wd, gs)
        return loss

    def _update_chunk(self, w, g, buf, beta, lr, wd, gscale=None) -> None:
        """``buf`` is on the same device as ``w`` here."""
        n, m = w.shape[-2], w.shape[-1]
        native = (w.is_cuda and w.dtype == torch.bfloat16 and w.is_contiguous() and g.is_contiguous()
                  and buf.is_contiguous() and w.numel() % 8 == 0 and g.dtype in (torch.float32, torch.bfloat16)
                  and buf.dtype in (torch.float32, torch.bfloat16))
        if native:
            L = _native.lib()
            upd = torch.empty(w.shape, dtype=torch.bfloat16, device=w.device)
            rc = L.pt_muon_momentum(g.data_ptr(), int(g.dtype == torch.float32), buf.data_ptr(),
                                    int(buf.dtype == torch.float32), upd.data_ptr(), w.numel(), float(beta),
                                    None if gscale is None else gscale.data_ptr(), _native.stream_ptr())
            _native.check(rc, "pt_muon_momentum")
        else:
            g32 = g.float() if gscale is None else g.float() * gscale.to(g.device)
            b32 = buf.float().lerp_(g32, 1 - beta)
            buf.copy_(b32)
            upd = g32.lerp(b32, beta)
        orth = zeropower_via_newtonschulz5(upd, steps=5)
        scale = muon_scale_factor(n, m)
        if native:
            orth = orth.contiguous()
            rc = _native.lib().pt_axpby_bf16(w.data_ptr(), orth.data_ptr(), w.numel(), float(1 - lr * wd),
                                             float(-lr * scale), _native.stream_ptr())
            _native.check(rc, "pt_axpby_bf16")
        else:
            w.mul_(1 - lr * wd)
            w.add_(orth.to(w.dtype), alpha=-lr * scale)

    def _run_offloaded(self, work, beta, lr, wd, tail=()) -> None:
        """Stream host-resident momentum chunks through three device staging buffers."""
        dev = work[0][0].device
        if self._streams is None:
            self._streams = (torch.cuda.Stream(device=dev), torch.cuda.Stream(device=dev))
        h2d, d2h = self._streams
        max_elems = max(item[0].numel() for item in work)
        if not self._stage or self._stage[0].numel() < max_elems:
            self._stage = [torch.empty(max_elems, dtype=self.momentum_dtype, device=dev) for _ in range(3)]
        comp = torch.cuda.current_stream(dev)
        free_ev = [None, None, None]  # d2h finished reading staging buffer k
        loaded = {}

        def prefetch(i):
            if i >= len(work):
                return
            k = i % 3
            w, _, st = work[i][:3]
            with torch.cuda.stream(h2d):
                if free_ev[k] is not None:
                    h2d.wait_event(free_ev[k])
                view = self._stage[k][: w.numel()].view(w.shape)
                view.copy_(st, non_blocking=True)
                ev = torch.cuda.Event()
                ev.record(h2d)
            loaded[i] = (view, ev)

        prefetch(0)
        prefetch(1)
        for i, (w, g, st, gs) in enumerate(work):
            view, ev = loaded.pop(i)
            comp.wait_event(ev)
            self._update_chunk(w, g, view, beta, lr, wd, gs)
            done = torch.cuda.Event()
            done.record(comp)
            with torch.cuda.stream(d2h):
                d2h.wait_event(done)
                st.copy_(view, non_blocking=True)
                fe = torch.cuda.Event()
                fe.record(d2h)
            free_ev[i % 3] = fe
            prefetch(i + 2)
        for w, g, st, gs in tail:
            self._update_chunk(w, g, st, beta, lr, wd, gs)
        comp.wait_stream(d2h)


class AdamW(torch.optim.Optimizer):
    """AdamW with fp32 moments over (possibly bf16) owner-sharded parameters; one fused kernel per
    parameter on CUDA."""

    def __init__(self, params, lr: float = 1e-3, betas=(0.9, 0.999), eps: float = 1e-8, weight_decay: float = 0.01):
        defaults = dict(lr=lr, betas=betas, eps=eps, weight_decay=weight_decay)
        super().__init__(params, defaults)

    @torch.no_grad()
    def step(self, closure=None):
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        for group in self.param_groups:
            lr, (b1, b2), eps, wd = group["lr"], group["betas"], group["eps"], group["weight_decay"]
            for p in group["params"]:
                g = _grad_of(p)
                if g is None or not _owned(p):
                    continue
                st = self.state[p]
                if len(st) == 0:
                    st["step"] = torch.zeros((), dtype=torch.float32)
                    st["exp_avg"] = torch.zeros(p.shape, dtype=torch.float32, device=p.device)
                    st["exp_avg_sq"] = torch.zeros(p.shape, dtype=torch.float32, device=p.device)
                st["step"] += 1
                t = float(st["step"])
                gs = _grad_scale_of(p)
                m, v = st["exp_avg"], st["exp_avg_sq"]
                bc1, bc2 = 1 - b1 ** t, 1 - b2 ** t
                if (p.is_cuda and p.is_contiguous() and g.is_contiguous() and p.numel() % 8 == 0
                        and p.dtype in (torch.float32, torch.bfloat16) and g.dtype in (torch.float32, torch.bfloat16)
                        and p.data_ptr() % 16 == 0 and g.data_ptr() % 16 == 0):
                    rc = _native.lib().pt_adamw(p.data_ptr(), int(p.dtype == torch.float32), g.data_ptr(),
                                                int(g.dtype == torch.float32), m.data_ptr(), v.data_ptr(), p.numel(),
                                                None if gs is None else gs.data_ptr(), float(lr), float(b1), float(b2), float(eps), float(wd),
                                                float(bc1), float(bc2), _native.stream_ptr())
                    _native.check(rc, "pt_adamw")
                    continue
                g32 = g.float() if gs is None else g.float() * gs.to(g.device)
                m.lerp_(g32, 1 - b1)
                v.mul_(b2).addcmul_(g32, g32, value=1 - b2)
                denom = (v / bc2).sqrt_().add_(eps)
                if p.dtype == torch.float32:
                    p.mul_(1 - lr * wd).addcdiv_(m, denom, value=-lr / bc1)
                else:
                    p32 = p.float().mul_(1 - lr * wd).addcdiv_(m, denom, value=-lr / bc1)
                    p.copy_(p32)
        return loss
