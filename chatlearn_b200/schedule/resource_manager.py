"""Resources of the job: the ranks (one per GPU), their nodes, and the bundles reserved for each role.

Parity: chatlearn/schedule/resource_manager.py:29-86, which reads Ray node resources
(``gpu_per_node``, ``cpu_per_node``) and builds one placement group per role: a role that fits
a node gets a single bundle ``{GPU: n, CPU: cpus * n / gpus}`` packed on one node, a larger role
gets whole-node bundles, a CPU-only role gets one bundle per entry of ``num_cpus``.  With one
process per GPU there is no scheduler to ask: the pool is the set of global ranks, grouped
into nodes by ``gpus_per_node``; ``create_placement_group`` reserves ranks under the same
rules (a bundle never straddles a node boundary, ``PACK`` fills a node before opening the
next, ``SPREAD`` rotates over nodes), and ``remove_placement_groups`` gives them back.  The
per-node CPU count comes from the operating system; the table of nodes (host name, GPU name and
memory per rank) is collected once over the process group and checked for uniformity.
"""
import os
import socket
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence

import torch
import torch.distributed as dist


@dataclass
class Bundle:
    """Ranks (and CPU cores) of one node reserved together."""
    node: int
    ranks: List[int]
    cpus: int = 0


@dataclass
class PlacementGroup:
    name: str
    bundles: List[Bundle]
    strategy: str = "PACK"
    state: str = "CREATED"

    @property
    def ranks(self) -> List[int]:
        return [r for b in self.bundles for r in b.ranks]

    @property
    def bundle_specs(self) -> List[Dict[str, int]]:
        return [{"GPU": len(b.ranks), "CPU": b.cpus} for b in self.bundles]


@dataclass
class NodeInfo:
    index: int
    host: str
    ranks: List[int]
    gpu_name: str = "cpu"
    gpu_mem_gib: float = 0.0
    cpus: int = 0
    free: List[int] = field(default_factory=list)      # ranks not reserved by a placement group


class ResourceManager:
    def __init__(self, models=None, gather_node_table: bool = False):
        self.models = list(models or [])
        self.name2models = {m.name: m for m in self.models}
        self.world_size = dist.get_world_size() if dist.is_initialized() else 1
        self.rank = dist.get_rank() if dist.is_initialized() else 0
        self.gpus_per_node = int(os.environ.get("GPUS_PER_NODE", os.environ.get(
            "LOCAL_WORLD_SIZE", str(self.world_size))))
        self.gpu_per_node = self.gpus_per_node          # the reference's attribute name
        self.cpu_per_node = os.cpu_count() or 1
        self.has_gpu = torch.cuda.is_available()
        self.nnode = (self.world_size + self.gpus_per_node - 1) // self.gpus_per_node
        self.total_gpu = self.world_size
        self.placement_groups: List[PlacementGroup] = []
        self.model_to_placegroup: Dict[str, PlacementGroup] = {}
        self._nodes = [NodeInfo(i, socket.gethostname() if i == self.rank // self.gpus_per_node else "", ranks,
                                cpus=self.cpu_per_node, free=list(ranks)) for i, ranks in enumerate(self.nodes())]
        if gather_node_table:
            self.gather_node_table()

    # ------------------------------------------------------------------ the pool
    @property
    def total_slots(self) -> int:
        """Ranks usable as "GPUs" (CPU ranks stand in for GPUs in gloo runs)."""
        return self.world_size

    def nodes(self) -> List[List[int]]:
        n = self.gpus_per_node
        return [list(range(s, min(s + n, self.world_size))) for s in range(0, self.world_size, n)]

    def node_of(self, rank: int) -> int:
        return rank // self.gpus_per_node

    def gather_node_table(self) -> List[NodeInfo]:
        """Collective over the world: host name, device name and memory of every rank (what ``ray.nodes()`` tells
        the reference).  Raises if the ranks of one node disagree on the host, or nodes differ in their GPU type."""
        if self.has_gpu:
            p = torch.cuda.get_device_properties(torch.cuda.current_device())
            mine = (socket.gethostname(), p.name, round(p.total_memory / 2 ** 30, 1), os.cpu_count() or 1)
        else:
            mine = (socket.gethostname(), "cpu", 0.0, os.cpu_count() or 1)
        table = [mine]
        if self.world_size > 1:
            table = [None] * self.world_size
            dist.all_gather_object(table, mine)
        for nd in self._nodes:
            rows = [table[r] for r in nd.ranks]
            hosts = {h for h, *_ in rows}
            if len(hosts) != 1:
                raise RuntimeError(f"ranks {nd.ranks} were expected on one node (gpus_per_node={self.gpus_per_node}) "
                                   f"but run on {sorted(hosts)}")
            nd.host, nd.gpu_name, nd.gpu_mem_gib, nd.cpus = rows[0]
        kinds = {nd.gpu_name for nd in self._nodes}
        if len(kinds) != 1:
            raise RuntimeError(f"nodes with different GPU types in one job: {sorted(kinds)}")
        return self._nodes

    # ------------------------------------------------------------------ placement groups
    def create_placement_group(self, num_gpus: int, num_cpus: Optional[Sequence[int]] = None, strategy: str = "PACK",
                               name: str = "") -> PlacementGroup:
        """Reserve ranks for a role.  ``num_gpus`` up to a node's size: one bundle on the node with the fewest free
        ranks that still fits (``PACK``) or the most (``SPREAD``); more: whole-node bundles, ``num_gpus`` must be a
        multiple of the node size.  ``num_gpus == 0``: CPU-only bundles of ``num_cpus[i]`` cores, no ranks reserved
        (CPU roles run on the ranks of GPU roles)."""
        assert strategy in ("PACK", "SPREAD")
        bundles: List[Bundle] = []
        if num_gpus > 0:
            per = self.gpus_per_node
            if num_gpus <= per:
                fits = [nd for nd in self._nodes if len(nd.free) >= num_gpus]
                if not fits:
                    raise RuntimeError(f"no node has {num_gpus} free GPUs left (free per node: "
                                       f"{[len(nd.free) for nd in self._nodes]})")
                nd = min(fits, key=lambda n: (len(n.free), n.index)) if strategy == "PACK" else \
                    max(fits, key=lambda n: (len(n.free), -n.index))
                ranks, nd.free = nd.free[:num_gpus], nd.free[num_gpus:]
                bundles.append(Bundle(nd.index, ranks, int(nd.cpus * num_gpus / per)))
            else:
                assert num_gpus % per == 0, f"a role larger than a node takes whole nodes ({num_gpus} % {per} != 0)"
                whole = [nd for nd in self._nodes if len(nd.free) == per]
                need = num_gpus // per
                if len(whole) < need:
                    raise RuntimeError(f"{need} whole nodes requested, {len(whole)} are free")
                for nd in whole[:need]:
                    bundles.append(Bundle(nd.index, list(nd.free), nd.cpus))
                    nd.free = []
        else:
            assert num_cpus is not None and isinstance(num_cpus, (list, tuple)), "num_cpus should be a list"
            for i, c in enumerate(num_cpus):
                bundles.append(Bundle(i % len(self._nodes), [], int(c)))
        pg = PlacementGroup(name or f"pg{len(self.placement_groups)}", bundles, strategy)
        self.placement_groups.append(pg)
        if name:
            self.model_to_placegroup[name] = pg
        return pg

    def reserve(self, name: str, ranks: Sequence[int]) -> PlacementGroup:
        """Record a placement that was computed elsewhere (colocated roles share ranks: the first role reserves
        them, the others reference the same bundles)."""
        by_node: Dict[int, List[int]] = {}
        for r in ranks:
            by_node.setdefault(self.node_of(r), []).append(r)
        bundles = []
        for n, rs in sorted(by_node.items()):
            nd = self._nodes[n]
            nd.free = [r for r in nd.free if r not in rs]
            bundles.append(Bundle(n, rs, int(nd.cpus * len(rs) / max(len(nd.ranks), 1))))
        pg = PlacementGroup(name, bundles, "PACK")
        self.placement_groups.append(pg)
        self.model_to_placegroup[name] = pg
        return pg

    def get_placement_group_state(self, pg: PlacementGroup) -> str:
        return pg.state

    def remove_placement_groups(self):
        for pg in self.placement_groups:
            for b in pg.bundles:
                nd = self._nodes[b.node]
                nd.free = sorted(set(nd.free) | set(b.ranks))
            pg.state = "REMOVED"
        self.placement_groups = []
        self.model_to_placegroup = {}
