"""(pp, dp, cp, ep) process mesh with explicit rank arithmetic.

Ranks are laid out outer-to-inner as (pp, dp, cp, ep), so the communication-heavy axes (expert
all-to-all, context-parallel KV exchange) are neighbours inside one NVLink/NVSwitch domain — the
ordering of pithtrain/modules/distributed.py:129-161 in the reference. Only the groups the
framework really uses are created: the four axis groups and three flattened ones
(dp×cp for expert-parameter sharding, dp×cp×ep for non-expert sharding, dp×ep for routing
statistics). Every rank creates every group in the same order, as ``new_group`` requires.
"""

from __future__ import annotations

import itertools
from dataclasses import dataclass, field
from typing import Dict, List, Sequence, Tuple

import torch.distributed as dist

AXES = ("pp", "dp", "cp", "ep")


@dataclass
class Mesh4D:
    pp: int
    dp: int
    cp: int
    ep: int
    rank: int
    groups: Dict[Tuple[str, ...], object] = field(default_factory=dict)
    group_ranks: Dict[Tuple[str, ...], List[int]] = field(default_factory=dict)

    @property
    def shape(self) -> Tuple[int, int, int, int]:
        return (self.pp, self.dp, self.cp, self.ep)

    @property
    def world_size(self) -> int:
        return self.pp * self.dp * self.cp * self.ep

    def coords(self, rank: int | None = None) -> Dict[str, int]:
        r = self.rank if rank is None else rank
        out = {}
        for name, size in reversed(list(zip(AXES, self.shape))):
            out[name] = r % size
            r //= size
        return out

    def rank_of(self, **coords: int) -> int:
        r = 0
        for name, size in zip(AXES, self.shape):
            r = r * size + coords[name]
        return r

    def ranks_along(self, axes: Sequence[str], rank: int | None = None) -> List[int]:
        """Ranks that share this rank's coordinates on every axis not in ``axes`` (mesh order)."""
        base = self.coords(rank)
        sizes = [dict(zip(AXES, self.shape))[a] for a in axes]
        out = []
        for combo in itertools.product(*[range(s) for s in sizes]):
            c = dict(base)
            c.update(dict(zip(axes, combo)))
            out.append(self.rank_of(**c))
        return out

    def all_groups_along(self, axes: Sequence[str]) -> List[List[int]]:
        seen, out = set(), []
        for r in range(self.world_size):
            g = tuple(self.ranks_along(axes, r))
            if g not in seen:
                seen.add(g)
                out.append(list(g))
        return out

    def build_groups(self, timeout=None) -> None:
        """Create the process groups (collective call: every rank, same order)."""
        wanted = [("pp",), ("dp",), ("cp",), ("ep",), ("dp", "cp"), ("dp", "cp", "ep"), ("dp", "ep")]
        for axes in wanted:
            mine = self.ranks_along(axes)
            self.group_ranks[axes] = mine
            if not dist.is_initialized() or self.world_size == 1:
                self.groups[axes] = None
                continue
            for ranks in self.all_groups_along(axes):
                kw = {"timeout": timeout} if timeout is not None else {}
                g = dist.new_group(ranks=ranks, **kw) if len(ranks) > 1 else None
                if ranks == mine:
                    self.groups[axes] = g

    def ensure_group(self, *axes: str):
        """Group along ``axes``, created on first use (collective: all ranks must call it)."""
        key = tuple(axes)
        if key not in self.groups:
            mine = self.ranks_along(key)
            self.group_ranks[key] = mine
            self.groups[key] = None
            if dist.is_initialized() and self.world_size > 1:
                for ranks in self.all_groups_along(key):
                    g = dist.new_group(ranks=ranks) if len(ranks) > 1 else None
                    if ranks == mine:
                        self.groups[key] = g
        return self.groups[key]

    def group(self, *axes: str):
        return self.groups.get(tuple(axes))

    def local_rank(self, *axes: str) -> int:
        return self.group_ranks[tuple(axes)].index(self.rank)

    def size(self, *axes: str) -> int:
        n = 1
        d = dict(zip(AXES, self.shape))
        for a in axes:
            n *= d[a]
        return n
