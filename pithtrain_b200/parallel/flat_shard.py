"""Flat, owner-sharded parameters: the framework's own ZeRO-style data parallelism.

The reference wraps modules in FSDP2 and then disables resharding and gradient sync for the whole
pipeline step, so in effect parameters are all-gathered once and gradients reduce-scattered once
per optimizer step (pithtrain/modules/training.py:328-376, pithtrain/dualpipe/dualpipev.py:513-525,
629-653). With 180 GB per GPU that steady state is simply kept resident:

* every parameter of a group lives in one flat bf16 buffer, every gradient accumulator in one flat
  buffer of ``grad_dtype``; parameters and ``main_grad`` are views, so GEMM epilogues accumulate
  weight gradients in place and the optimizer runs over few large tensors;
* the buffer is cut into one region per rank of the shard group and whole parameters (never
  slices) are assigned to regions by greedy size balancing. The owner of a region receives the
  reduced gradients of its parameters (one ``reduce_scatter`` over the flat buffer), runs the
  optimizer for them — Muon's Newton-Schulz sees full matrices without any gather — and the updated
  regions are all-gathered back into every rank's flat parameter buffer;
* optimizer state exists only on the owner, so it is sharded like ZeRO-1/2/3 state;
* with ``reshard_params`` the parameters are sharded too between steps: after the gradient reduction a rank frees the
  regions it does not own (optimizer step, checkpoint staging and anything else between steps then run with
  ``1/group_size`` of the group's parameters resident) and the next step starts with one all-gather.

Expert parameters shard over dp×cp, everything else over dp×cp×ep, like the reference's FSDP meshes.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence, Tuple

import torch
import torch.distributed as dist
import torch.nn as nn

from ..ops.linear import FusedWeights

ALIGN_ELEMS = 128  # region and unit alignment: 256 B for bf16, keeps TMA/vector accesses aligned


@dataclass
class Unit:
    """A block that is placed contiguously and owned by one rank: one parameter or a fused set."""

    names: List[str]
    params: List[nn.Parameter]
    fused: Optional[FusedWeights] = None
    owner: int = 0
    offset: int = 0  # element offset inside the flat buffers

    @property
    def numel(self) -> int:
        return sum(p.numel() for p in self.params)

    @property
    def padded(self) -> int:
        return (self.numel + ALIGN_ELEMS - 1) // ALIGN_ELEMS * ALIGN_ELEMS


def collect_units(named_params: Sequence[Tuple[str, nn.Parameter]], fusions: Sequence[FusedWeights]) -> List[Unit]:
    by_id = {id(p): n for n, p in named_params}
    used = set()
    units: List[Unit] = []
    for fw in fusions:
        if all(id(p) in by_id for p in fw.params):
            units.append(Unit([by_id[id(p)] for p in fw.params], list(fw.params), fused=fw))
            used.update(id(p) for p in fw.params)
    for n, p in named_params:
        if id(p) not in used:
            units.append(Unit([n], [p]))
    return units


def assign_owners(units: List[Unit], group_size: int) -> List[int]:
    """Greedy balance (largest first onto the least-loaded rank). Deterministic on every rank.

    Returns the load (padded elements) per rank.
    """
    loads = [0] * group_size
    order = sorted(range(len(units)), key=lambda i: (-units[i].padded, units[i].names[0]))
    for i in order:
        r = min(range(group_size), key=lambda j: (loads[j], j))
        units[i].owner = r
        loads[r] += units[i].padded
    return loads


class FlatShardGroup:
    def __init__(self, name: str, named_params: Sequence[Tuple[str, nn.Parameter]], fusions: Sequence[FusedWeights],
                 group=None, group_size: int = 1, group_rank: int = 0, grad_dtype: torch.dtype = torch.float32,
                 replica_group=None, replica_size: int = 1, device=None, param_swapper=None,
                 fused_collectives: bool = True, reshard_params: bool = False) -> None:
        self.name = name
        # reshard_params: between the gradient reduction of one step and the start of the next, a rank keeps only the
        # parameters it owns; the regions of the other owners are freed and gathered again when the next step (or a
        # checkpoint save) needs them. That is parameter sharding in the form the reference runs it: FSDP2 with
        # resharding switched off inside a pipeline step, i.e. one gather per step
        # (pithtrain/modules/training.py:328-376, pithtrain/dualpipe/dualpipev.py:513-525,629-653).
        self.reshard_params = bool(reshard_params) and group_size > 1
        self.own_param: Optional[torch.Tensor] = None
        self.group, self.group_size, self.group_rank = group, group_size, group_rank
        self.replica_group, self.replica_size = replica_group, replica_size
        self.grad_divisor = 1
        self.defer_grad_scale = True
        self.grad_scale: Optional[torch.Tensor] = None  # pending factor on the accumulated gradients (device, [1])
        self.units = collect_units(named_params, fusions)
        self.named_params = list(named_params)
        if not self.units:
            self.region = 0
            self.flat_param = self.flat_grad = None
            return
        p0 = self.units[0].params[0]
        self.param_dtype = p0.dtype
        self.grad_dtype = grad_dtype
        device = device or p0.device
        if torch.device(device).type == "meta":
            raise ValueError("FlatShardGroup needs a real device for parameters built on the meta device")
        loads = assign_owners(self.units, group_size)
        self.region = max(max(loads), ALIGN_ELEMS)
        cursor = [r * self.region for r in range(group_size)]
        for u in sorted(self.units, key=lambda u: (u.owner, u.names[0])):
            u.offset = cursor[u.owner]
            cursor[u.owner] += u.padded
        total = self.region * group_size
        self.comm = None
        self._fused_sumsq = None
        if fused_collectives and not self.reshard_params and group_size > 1 and torch.device(device).type == "cuda":
            from . import fsdp_fused

            if fsdp_fused.usable(group, group_size, device):
                # buffers live in symmetric memory: peers read gradient regions and write parameter
                # regions directly, no NCCL reduce-scatter / all-gather
                self.comm = fsdp_fused.FusedShardComm(group, group_size, group_rank, self.region, self.param_dtype,
                                                      grad_dtype, device)
        if self.comm is not None:
            self.flat_param, self.flat_grad = self.comm.flat_param, self.comm.flat_grad
        else:
            self.flat_param = torch.zeros(total, dtype=self.param_dtype, device=device)
            self.flat_grad = torch.zeros(total, dtype=grad_dtype, device=device)
        if self.reshard_params:
            # owned parameters live in a buffer of their own, which persists; the flat buffer holds the others' regions
            # (and, while allocated, a copy of this rank's) and can be released
            self.own_param = torch.zeros(self.region, dtype=self.param_dtype, device=device)
        replaced: Dict[int, nn.Parameter] = {}

        def swap(old: nn.Parameter, new: nn.Parameter) -> None:
            replaced[id(old)] = new
            if param_swapper is not None:
                param_swapper(old, new)

        with torch.no_grad():
            for u in self.units:
                n = u.numel
                pv, gv = self.flat_param[u.offset:u.offset + n], self.flat_grad[u.offset:u.offset + n]
                if self.own_param is not None and u.owner == group_rank:
                    lo = u.offset - group_rank * self.region
                    pv = self.own_param[lo:lo + n]
                if u.fused is not None:
                    u.fused.rebind(pv, gv, copy=True, swap=swap)
                    u.params = list(u.fused.params)
                else:
                    p = u.params[0]
                    if p.is_meta:
                        q = nn.Parameter(pv.view(p.shape), requires_grad=p.requires_grad)
                        for attr in ("_init_fill", "_init_fn"):
                            if hasattr(p, attr):
                                setattr(q, attr, getattr(p, attr))
                        swap(p, q)
                        u.params[0] = p = q
                    else:
                        pv.view(p.shape).copy_(p.data)
                        p.data = pv.view(p.shape)
                    p.main_grad = gv.view(p.shape)
                for p in u.params:
                    p.grad = None
                    p._shard_owner = u.owner
                    p._shard_group = self
        self.named_params = [(n, replaced.get(id(p), p)) for n, p in self.named_params]

    # ------------------------------------------------------------------ views
    def my_slice(self, flat: torch.Tensor) -> torch.Tensor:
        return flat[self.group_rank * self.region:(self.group_rank + 1) * self.region]

    def owned_params(self) -> List[Tuple[str, nn.Parameter]]:
        out = []
        for u in self.units:
            if u.owner == self.group_rank:
                out.extend(zip(u.names, u.params))
        return out

    def is_owned(self, p: nn.Parameter) -> bool:
        return getattr(p, "_shard_owner", self.group_rank) == self.group_rank

    # ------------------------------------------------------------------ step protocol
    def fold_autograd_grads(self) -> None:
        """Move gradients that plain autograd left in ``.grad`` into the flat accumulators."""
        for _, p in self.named_params:
            if p.grad is not None:
                p.main_grad.add_(p.grad.to(p.main_grad.dtype))
                p.grad = None

    def apply_clip(self, coef: torch.Tensor) -> None:
        """Scale the owned gradients by the clip coefficient (folded into ``grad_scale`` when deferred)."""
        if self.flat_grad is None:
            return
        if self.grad_scale is not None:
            self.grad_scale = self.grad_scale * coef.to(torch.float32).reshape(1)
        else:
            self.my_slice(self.flat_grad).mul_(coef.to(self.flat_grad.dtype))

    def zero_grad(self) -> None:
        self.grad_scale = None
        if self.flat_grad is not None:
            if self.comm is not None:
                self.comm.before_zero_grad()  # owners may still be reading this rank's gradients
            self.flat_grad.zero_()

    def scale_grads(self, scale) -> None:
        """Multiply accumulated gradients by ``scale / grad_divisor``.

        ``grad_divisor`` is the number of ranks whose tokens reached these parameters without being
        averaged by :meth:`reduce_grads`: ``ep`` for expert parameters (every expert-parallel rank
        feeds its own micro-batches into each expert, and expert gradients are only averaged over
        dp×cp), 1 for the rest. With it every parameter receives the gradient of the same global
        token-mean loss on every mesh. (The reference leaves expert gradients ``ep`` times larger,
        pithtrain/tasks/pretrain_lm.py:393-396 together with the dp×cp expert mesh of
        pithtrain/modules/training.py:364-370.)
        """
        if self.flat_grad is None:
            return
        scale = scale / self.grad_divisor if self.grad_divisor != 1 else scale
        if self.flat_grad.is_cuda and self.defer_grad_scale:
            # no pass over the gradients: the factor travels to the optimizer kernels as a device scalar
            # (grad_scale) and the norm is corrected by its square
            s = torch.as_tensor(scale, dtype=torch.float32, device=self.flat_grad.device).reshape(1)
            self.grad_scale = s if self.grad_scale is None else self.grad_scale * s
        else:
            self.flat_grad.mul_(scale)

    def reduce_grads(self) -> None:
        """Average gradients over the shard group; afterwards only this rank's region is meaningful."""
        if self.flat_grad is None:
            return
        self._fused_sumsq = None
        if self.group_size > 1 and self.comm is not None:
            sumsq = self.comm.reduce_scatter(1.0)
            if self.replica_size == 1:
                self._fused_sumsq = sumsq  # the reduction pass already measured the owned region
        elif self.group_size > 1:
            mine = self.my_slice(self.flat_grad)
            backend = dist.get_backend(self.group)
            if backend == "nccl":
                dist.reduce_scatter_tensor(mine, self.flat_grad, op=dist.ReduceOp.AVG, group=self.group)
            else:
                chunks = list(self.flat_grad.view(self.group_size, self.region).unbind(0))
                out = torch.empty_like(mine)
                dist.reduce_scatter(out, [c.contiguous() for c in chunks], group=self.group)
                mine.copy_(out / self.group_size)
        if self.replica_size > 1:
            mine = self.my_slice(self.flat_grad)
            dist.all_reduce(mine, group=self.replica_group)
            mine.div_(self.replica_size)

    def owned_grad_sumsq(self) -> torch.Tensor:
        """Sum of squares of this rank's reduced gradients (with any pending scale applied)."""
        raw = self._owned_grad_sumsq_raw()
        if self.grad_scale is not None:
            raw = raw.to(self.grad_scale.device) * (self.grad_scale[0] * self.grad_scale[0])
        return raw

    def _owned_grad_sumsq_raw(self) -> torch.Tensor:
        if self.flat_grad is None:
            return torch.zeros((), dtype=torch.float32)
        if self._fused_sumsq is not None:
            out, self._fused_sumsq = self._fused_sumsq, None
            return out
        g = self.my_slice(self.flat_grad)
        if g.is_cuda and g.dtype in (torch.float32, torch.bfloat16) and g.numel() % 8 == 0:
            from .. import _native

            L = _native.lib()
            part = torch.empty(L.pt_sumsq_grid(), dtype=torch.float64, device=g.device)
            rc = L.pt_sumsq(g.data_ptr(), int(g.dtype == torch.float32), g.numel(), part.data_ptr(), _native.stream_ptr())
            _native.check(rc, "pt_sumsq")
            return part.sum().float() / self.replica_size
        total = torch.zeros((), dtype=torch.float32, device=g.device)
        for c in g.split(1 << 26):
            total += c.float().pow(2).sum()
        return total / self.replica_size

    def params_resident(self) -> bool:
        return self.flat_param is None or self.flat_param.untyped_storage().size() > 0

    def release_params(self) -> None:
        """Free the regions of the other owners (``reshard_params`` only; the owned parameters are elsewhere)."""
        if self.reshard_params and self.flat_param is not None and self.params_resident():
            self.flat_param.untyped_storage().resize_(0)

    def ensure_params(self) -> None:
        """Make every parameter of the group readable again after :meth:`release_params`."""
        if self.reshard_params and self.flat_param is not None and not self.params_resident():
            self.flat_param.untyped_storage().resize_(self.flat_param.numel() * self.flat_param.element_size())
            self.gather_params()

    def gather_params(self) -> None:
        """Publish the owners' updated regions to every rank of the shard group."""
        if self.flat_param is None or self.group_size == 1:
            return
        if self.comm is not None:
            self.comm.push_params()
            return
        if self.reshard_params and not self.params_resident():
            return  # stays sharded; ensure_params gathers when the parameters are needed
        mine = self.own_param if self.own_param is not None else self.my_slice(self.flat_param)
        backend = dist.get_backend(self.group)
        if backend == "nccl":
            dist.all_gather_into_tensor(self.flat_param, mine, group=self.group)
        else:
            outs = [torch.empty_like(mine) for _ in range(self.group_size)]
            dist.all_gather(outs, mine.contiguous(), group=self.group)
            self.flat_param.copy_(torch.cat(outs))

    def wait_params(self) -> None:
        """Order later work of this stream after the arrival of every peer's published region."""
        if self.comm is not None:
            self.comm.before_forward()

    # ------------------------------------------------------------------ reporting
    def nbytes(self) -> int:
        if self.flat_param is None:
            return 0
        own = 0 if self.own_param is None else self.own_param.numel() * self.own_param.element_size()
        return own + self.flat_param.numel() * self.flat_param.element_size() + self.flat_grad.numel() * self.flat_grad.element_size()


def find_fusions(module: nn.Module) -> List[FusedWeights]:
    out = []
    for m in module.modules():
        for v in vars(m).values():
            if isinstance(v, FusedWeights):
                out.append(v)
    return out


def is_expert_param(name: str) -> bool:
    return ".experts." in name


def build_shard_groups(module: nn.Module, *, expert_group=None, expert_group_size: int = 1, expert_group_rank: int = 0,
                       dense_group=None, dense_group_size: int = 1, dense_group_rank: int = 0,
                       grad_dtype: torch.dtype = torch.float32, expert_replica=(None, 1), dense_replica=(None, 1),
                       prefix: str = "", device=None, expert_grad_divisor: int = 1,
                       reshard_params: bool = False) -> List[FlatShardGroup]:
    """Create the two shard groups (experts, everything else) of one model chunk."""
    named = [(prefix + n, p) for n, p in module.named_parameters() if p.requires_grad]
    fusions = find_fusions(module)
    home = {}
    for m in module.modules():
        for k, p in m._parameters.items():
            if p is not None:
                home[id(p)] = (m, k)

    def param_swapper(old: nn.Parameter, new: nn.Parameter) -> None:
        m, k = home[id(old)]
        m._parameters[k] = new
        home[id(new)] = (m, k)

    ex = [(n, p) for n, p in named if is_expert_param(n)]
    de = [(n, p) for n, p in named if not is_expert_param(n)]
    ex_ids = {id(p) for _, p in ex}
    ex_f = [f for f in fusions if id(f.params[0]) in ex_ids]
    de_f = [f for f in fusions if id(f.params[0]) not in ex_ids]
    groups = []
    if de:
        groups.append(FlatShardGroup(prefix + "dense", de, de_f, dense_group, dense_group_size, dense_group_rank,
                                     grad_dtype, dense_replica[0], dense_replica[1], device=device,
                                     param_swapper=param_swapper, reshard_params=reshard_params))
    if ex:
        groups.append(FlatShardGroup(prefix + "experts", ex, ex_f, expert_group, expert_group_size, expert_group_rank,
                                     grad_dtype, expert_replica[0], expert_replica[1], device=device,
                                     param_swapper=param_swapper, reshard_params=reshard_params))
        groups[-1].grad_divisor = max(int(expert_grad_divisor), 1)
    return groups
