from .engine import RolloutEngine, SamplingParams
from .scheduler import BlockAllocator, Scheduler, Sequence
