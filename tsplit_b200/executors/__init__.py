"""Executor family (base, stream, multi-stream and the memory-saving ones)."""
from .base import Executor, StreamExecutor, MultiStreamExecutor

__all__ = ["Executor", "StreamExecutor", "MultiStreamExecutor"]
