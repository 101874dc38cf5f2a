"""Resources of the job: the ranks (one per GPU) and their nodes.

Parity: chatlearn/schedule/resource_manager.py:29-86, which reads Ray node
resources and builds placement groups.  With one process per GPU the resource
pool is the set of global ranks; ``gpus_per_node`` groups them into nodes so a
model-parallel group never straddles a node boundary by accident.
"""
import os
from typing import List

import torch
import torch.distributed as dist


class ResourceManager:
    def __init__(self, models=None):
        self.models = models or []
        self.world_size = dist.get_world_size() if dist.is_initialized() else 1
        self.rank = dist.get_rank() if dist.is_initialized() else 0
        self.gpus_per_node = int(os.environ.get("GPUS_PER_NODE", os.environ.get(
            "LOCAL_WORLD_SIZE", str(self.world_size))))
        self.has_gpu = torch.cuda.is_available()

    @property
    def total_slots(self) -> int:
        """Ranks usable as "GPUs" (CPU ranks stand in for GPUs in gloo runs)."""
        return self.world_size

    def nodes(self) -> List[List[int]]:
        n = self.gpus_per_node
        return [list(range(s, min(s + n, self.world_size))) for s in range(0, self.world_size, n)]
