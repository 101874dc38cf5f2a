from .context_parallel import ContextParallel, zigzag_indices
from .expert_parallel import ExpertParallel
from .groups import Group, new_group, single_group
from .mesh import Mesh, build_mesh
from .ulysses import UlyssesGroup
