from .engine import AsyncRollout, RolloutEngine, RolloutSession, SamplingParams
from .scheduler import BlockAllocator, Scheduler, Sequence
