"""tsplit_b200 — a Blackwell-native define-then-run training framework with the
capabilities of the TSplit / "Athena" reference: graph construction and
autodiff, memory-saving executors (vDNN, SuperNeurons, recompute, Capuchin,
TSplit micro-tensor planning), hand-written sm_100a kernels and NVSwitch
data-parallel training.

    from tsplit_b200 import ndarray, gpu_ops as ad, optimizer
"""
from . import ndarray, stream, graph, optimizer, model, metrics, logger    # noqa: F401
from . import profiler, gpu_memory_manager, graphboard                     # noqa: F401
from . import gpu_ops                                                       # noqa: F401
from . import communicator                                                  # noqa: F401

__version__ = "0.1.0"
