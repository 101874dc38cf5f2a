"""Rank → (tp, cp, dp, pp, ep) coordinates and the process groups between them.

Layout (fastest to slowest): ``tp, cp, dp, pp`` for dense parameters and
``etp, ep, edp, pp`` for expert parameters, the convention the reference obtains
from Megatron-Core ``parallel_state`` (sizes validated in
chatlearn/configs/megatron_config.py:344-371).  One instance is built per model
role over the role's rank set, so a trainer at TP2·EP4 and a rollout engine at
TP2 × 4 replicas coexist in one job.
"""
from dataclasses import dataclass, field
from typing import Dict, List

import torch.distributed as dist

from .groups import Group, new_group, single_group


@dataclass
class Mesh:
    ranks: List[int]                       # global ranks of this role, in role order
    tp: int = 1
    cp: int = 1
    pp: int = 1
    ep: int = 1
    etp: int = 1
    sp: int = 1                            # Ulysses (inside dp)
    shard: int = 0                         # hybrid sharding: ranks per shard group inside dp (0 = all of dp)
    groups: Dict[str, Group] = field(default_factory=dict)
    coords: Dict[str, int] = field(default_factory=dict)

    @property
    def world(self) -> int:
        return len(self.ranks)

    @property
    def dp(self) -> int:
        return self.world // (self.tp * self.cp * self.pp)

    @property
    def edp(self) -> int:
        return self.world // (self.etp * self.ep * self.pp)

    def coord_of(self, role_rank: int) -> Dict[str, int]:
        r = role_rank
        c = {}
        c["tp"], r = r % self.tp, r // self.tp
        c["cp"], r = r % self.cp, r // self.cp
        c["dp"], r = r % self.dp, r // self.dp
        c["pp"] = r
        e = role_rank % (self.world // self.pp)
        c["etp"], e = e % self.etp, e // self.etp
        c["ep"], e = e % self.ep, e // self.ep
        c["edp"] = e
        c["sp"] = c["dp"] % self.sp
        c["dp_outer"] = c["dp"] // self.sp
        shard = self.shard or self.dp
        c["dp_shard"], c["dp_rep"] = c["dp"] % shard, c["dp"] // shard
        return c

    def group_ranks(self, kind: str) -> List[List[int]]:
        """All groups of ``kind`` as lists of role-local ranks."""
        keys = {"tp": ("cp", "dp", "pp"), "cp": ("tp", "dp", "pp"), "dp": ("tp", "cp", "pp"),
                "pp": ("tp", "cp", "dp"), "ep": ("etp", "edp", "pp"), "etp": ("ep", "edp", "pp"),
                "edp": ("etp", "ep", "pp"), "sp": ("tp", "cp", "dp_outer", "pp"),
                "dp_cp": ("tp", "pp"), "mp": ("dp",), "dp_outer": ("tp", "cp", "sp", "pp"),
                # hybrid sharding: neighbours in dp form a shard group, ranks with the same place in their shard
                # group form a replica group
                "dp_shard": ("tp", "cp", "dp_rep", "pp"), "dp_rep": ("tp", "cp", "dp_shard", "pp")}[kind]
        buckets: Dict[tuple, List[int]] = {}
        for r in range(self.world):
            c = self.coord_of(r)
            buckets.setdefault(tuple(c[k] for k in keys), []).append(r)
        return list(buckets.values())


def build_mesh(ranks: List[int], tp=1, cp=1, pp=1, ep=1, etp=1, sp=1,
               kinds=("tp", "cp", "dp", "pp", "ep", "edp", "sp", "dp_cp", "mp"), shard=0) -> Mesh:
    """Create the process groups of a role.  Collective over the *whole job*:
    every rank of the job must call it with identical arguments (ranks outside
    ``ranks`` take part in group creation only)."""
    m = Mesh(list(ranks), tp, cp, pp, ep, etp, sp, shard)
    assert m.world % (tp * cp * pp) == 0 and m.world % (etp * ep * pp) == 0
    assert not shard or m.dp % shard == 0, "the shard group size must divide the data-parallel size"
    assert m.dp % sp == 0, "Ulysses size must divide the data-parallel size"
    me = dist.get_rank() if dist.is_initialized() else 0
    role_rank = m.ranks.index(me) if me in m.ranks else -1
    if role_rank >= 0:
        m.coords = m.coord_of(role_rank)
    for kind in kinds:
        for local in m.group_ranks(kind):
            glob = [m.ranks[i] for i in local]
            if len(glob) == 1 or not dist.is_initialized():
                g = single_group() if me in glob else None
                if g is not None:
                    g.ranks = glob
            else:
                g = new_group(glob, f"{kind}")
            if g is not None and me in glob:
                m.groups[kind] = g
    return m
