"""Host layer of the engine: same classes and method names as the reference's ``engine/`` package."""
from .sampling_params import SamplingParams
from .sequence import Sequence, SequenceStatus
from .block_manager import BlockManager, NativeBlockManager
from .scheduler import Scheduler

__all__ = ["SamplingParams", "Sequence", "SequenceStatus", "BlockManager", "NativeBlockManager", "Scheduler"]
