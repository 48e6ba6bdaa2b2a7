"""Executor family (base, stream, multi-stream and the memory-saving ones)."""
from .base import Executor, StreamExecutor, MultiStreamExecutor
from .engine import MemoryExecutor
from .policies import vdnnExecutor, recomputeExecutor, superNeuronsExecutor, capuchinExecutor
from .profile import profileExecutor
from .microop import microopExecutor, microopPlanner, microopOptimizer, max_batch_search

__all__ = ["Executor", "StreamExecutor", "MultiStreamExecutor", "MemoryExecutor", "vdnnExecutor",
           "recomputeExecutor", "superNeuronsExecutor", "capuchinExecutor", "profileExecutor", "microopExecutor", "microopPlanner",
           "microopOptimizer", "max_batch_search"]
