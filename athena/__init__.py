"""Drop-in import name for code written against the reference:

    from athena import ndarray, gpu_ops as ad, optimizer
    from athena.microopOptimizer import microopOptimizer
    from athena.microopPlanner import microopPlanner

Every submodule is the ``tsplit_b200`` one."""
import sys as _sys
import types as _types

import tsplit_b200 as _t
from tsplit_b200 import (ndarray, stream, graph, optimizer, model, metrics, gpu_ops, logger, profiler,  # noqa: F401
                         gpu_memory_manager, communicator, graphboard)
from tsplit_b200.executors.microop import microopOptimizer as _opt, microopPlanner as _plan

for _n in ("ndarray", "stream", "graph", "optimizer", "model", "metrics", "gpu_ops", "logger", "profiler",
           "gpu_memory_manager", "communicator", "graphboard"):
    _sys.modules["athena." + _n] = getattr(_t, _n)
for _n, _obj in (("microopOptimizer", _opt), ("microopPlanner", _plan)):
    _m = _types.ModuleType("athena." + _n)
    setattr(_m, _n, _obj)
    _sys.modules["athena." + _n] = _m
    globals()[_n] = _m
