"""Rank layout for data x pipeline x tensor parallelism on one NVSwitch domain.

Global rank = ((dp_idx * pp) + pp_idx) * tp + tp_idx: the tensor-parallel ranks of one stage are
adjacent (they exchange the most data; over NVSwitch every pair has the same bandwidth, so this
only matters for readability), pipeline neighbours are ``tp`` ranks apart.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional

import torch.distributed as dist


@dataclass
class Topology:
    world: int
    rank: int
    tp: int = 1
    pp: int = 1
    dp: int = 1
    tp_group: Optional[dist.ProcessGroup] = None
    pp_group: Optional[dist.ProcessGroup] = None
    dp_group: Optional[dist.ProcessGroup] = None

    @property
    def tp_idx(self) -> int:
        return self.rank % self.tp

    @property
    def pp_idx(self) -> int:
        return (self.rank // self.tp) % self.pp

    @property
    def dp_idx(self) -> int:
        return self.rank // (self.tp * self.pp)

    def rank_of(self, dp_idx: int, pp_idx: int, tp_idx: int) -> int:
        return (dp_idx * self.pp + pp_idx) * self.tp + tp_idx

    @property
    def prev_stage_rank(self) -> Optional[int]:
        return self.rank_of(self.dp_idx, self.pp_idx - 1, self.tp_idx) if self.pp_idx > 0 else None

    @property
    def next_stage_rank(self) -> Optional[int]:
        return self.rank_of(self.dp_idx, self.pp_idx + 1, self.tp_idx) if self.pp_idx < self.pp - 1 else None


def groups_for(world: int, tp: int, pp: int) -> dict:
    """Pure function (testable without a process group): rank lists of every TP / PP / DP group."""
    assert world % (tp * pp) == 0
    dp = world // (tp * pp)
    tp_groups = [[(d * pp + p) * tp + t for t in range(tp)] for d in range(dp) for p in range(pp)]
    pp_groups = [[(d * pp + p) * tp + t for p in range(pp)] for d in range(dp) for t in range(tp)]
    dp_groups = [[(d * pp + p) * tp + t for d in range(dp)] for p in range(pp) for t in range(tp)]
    return {"tp": tp_groups, "pp": pp_groups, "dp": dp_groups, "dp_size": dp}


def build_topology(tp: int = 1, pp: int = 1) -> Topology:
    """Collective: every rank must call it (creates all subgroups in the same order)."""
    world, rank = dist.get_world_size(), dist.get_rank()
    g = groups_for(world, tp, pp)
    topo = Topology(world, rank, tp, pp, g["dp_size"])
    for kind in ("tp", "pp", "dp"):
        for ranks in g[kind]:
            grp = dist.new_group(ranks) if len(ranks) > 1 else None
            if rank in ranks:
                setattr(topo, f"{kind}_group", grp)
    return topo
