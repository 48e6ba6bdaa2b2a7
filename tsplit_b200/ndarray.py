"""Tensor container and device contexts.

Capability parity with the reference's ``python/athena/ndarray.py:9-455``
(``DLContext``, ``NDArray``, ``array``/``empty``, swap events, micro-tensor
slicing, the input/output overlap allocation) on a different substrate: storage
is a ``torch.Tensor`` (fp32) that is either a plain torch allocation or a view
into a capped arena handed out by the native pool (``runtime/pool.py``).

Layout rule: every 4-D array that lives on a GPU is stored channels-last
(logical NCHW shape, physical NHWC strides) because the tensor-core convolution
kernels read K-major (channel-contiguous) tiles.  Logical indexing, ``asnumpy``
and ``shape`` are unaffected.

Device types: 1 = CPU, 2 = GPU, 3 = simulated GPU (host storage, NumPy math,
capped pool) used to exercise the memory executors and the planner without a
GPU.
"""
from __future__ import annotations

import numpy as np
import torch

from .stream import Event

__all__ = [
    "DLContext", "NDArray", "cpu", "gpu", "simgpu", "is_gpu_ctx", "array", "empty",
    "tensor_reuse", "slice_for_micro_tensor", "split_shape", "ND_Sparse_Array",
    "sparse_array", "set_pool", "get_pool", "OutOfHBMBudget",
]


class OutOfHBMBudget(MemoryError):
    """Raised when an allocation does not fit the HBM budget of the active pool.

    The reference aborts with ``assert`` ("GPU available memory is not enough!",
    ``python/athena/gpu_ops/vdnnExecutor.py:332-333``); a typed error lets the
    batch-size sweep terminate cleanly."""


class OutOfHostSwapSpace(OutOfHBMBudget):
    """Raised when the pinned host buffers that hold swapped-out tensors would exceed the host swap budget
    (``TSPLIT_HOST_SWAP_GIB``, default: half of the host memory available when the executor plans).  Page-locked
    memory cannot be paged out, so an unbounded swap-everything policy at a very large batch would otherwise end
    with the process killed by the host's out-of-memory handler instead of an error a batch sweep can catch."""


def host_swap_budget_bytes():
    import os
    v = os.environ.get("TSPLIT_HOST_SWAP_GIB")
    if v:
        return int(float(v) * 2**30)
    try:
        import psutil
        return int(psutil.virtual_memory().available // 2)
    except Exception:
        return 64 << 30


class DLContext(object):
    MASK2STR = {1: "cpu", 2: "gpu", 3: "simgpu"}

    def __init__(self, device_id=0, device_type=1):
        self.device_id = int(device_id)
        self.device_type = int(device_type)

    def __repr__(self):
        return "%s(%d)" % (DLContext.MASK2STR[self.device_type], self.device_id)

    def __eq__(self, other):
        return isinstance(other, DLContext) and (self.device_id, self.device_type) == (
            other.device_id, other.device_type)

    def __hash__(self):
        return hash((self.device_id, self.device_type))

    @property
    def torch_device(self):
        if self.device_type == 2:
            return torch.device("cuda", self.device_id)
        return torch.device("cpu")


def cpu(dev_id=0):
    return DLContext(dev_id, 1)


def gpu(dev_id=0):
    return DLContext(dev_id, 2)


def simgpu(dev_id=0):
    """Host-backed stand-in for a GPU: same executor code paths, NumPy kernels."""
    return DLContext(dev_id, 3)


def is_gpu_ctx(ctx):
    return bool(ctx) and ctx.device_type in (2, 3)


def is_cuda_ctx(ctx):
    return bool(ctx) and ctx.device_type == 2


# ----------------------------------------------------------------------------
# active pool per context (None = plain torch allocations, no cap)
_POOLS = {}


def set_pool(ctx, pool):
    """Route every subsequent ``empty(..., ctx)`` through ``pool`` (or back to
    plain torch allocations with ``None``)."""
    if pool is None:
        _POOLS.pop(ctx, None)
    else:
        _POOLS[ctx] = pool


def get_pool(ctx):
    return _POOLS.get(ctx)


def _numel(shape):
    n = 1
    for s in shape:
        n *= int(s)
    return n


def _cl_strides(shape):
    n, c, h, w = shape
    return (h * w * c, 1, w * c, c)


def _make_view(flat, shape, channels_last):
    """View a flat fp32 tensor as ``shape`` (channels-last strides for 4-D)."""
    shape = tuple(int(s) for s in shape)
    if channels_last and len(shape) == 4:
        return flat.as_strided(shape, _cl_strides(shape))
    return flat.view(shape)


class NDArray(object):
    """Buffer object: no arithmetic, only storage, copies, swap state and
    micro-tensor views."""

    def __init__(self, tensor, ctx, block=None, pool=None, owns=True):
        self.t = tensor
        self.ctx = ctx
        self._shape = tuple(tensor.shape) if tensor is not None else ()
        self._block = block          # pool block id (None = torch-owned)
        self._pool = pool
        self._owns = owns
        self.swap = False
        self.in_gpu = tensor is not None
        self.splitted = False
        self.sTensor = []
        self.split_number = 1
        self.split_dimension = None
        if is_gpu_ctx(ctx):
            self.cpu2gpu_event = Event(ctx)
            self.gpu_event = Event(ctx)
            self.gpu2cpu_event = Event(ctx)

    # -- basic properties ------------------------------------------------
    @property
    def shape(self):
        return self._shape

    @property
    def handle(self):
        """Opaque handle kept for API compatibility (the tensor itself)."""
        return self.t

    @property
    def ptr(self):
        return self.t.data_ptr()

    @property
    def strides(self):
        return tuple(self.t.stride())

    @property
    def nbytes(self):
        return _numel(self._shape) * 4

    @property
    def is_cuda(self):
        return self.ctx.device_type == 2

    def is_channels_last(self):
        return len(self._shape) == 4 and self.strides == _cl_strides(self._shape)

    def is_contiguous(self):
        return self.t.is_contiguous()

    def same_layout(self, other):
        return self._shape == other._shape and self.strides == other.strides

    def is_dense(self):
        """True when the elements occupy one gap-free memory range (any order)."""
        t = self.t
        return t.is_contiguous() or (t.dim() == 4 and t.is_contiguous(memory_format=torch.channels_last))

    def __del__(self):
        try:
            self._release()
        except Exception:
            pass

    def _release(self):
        if self._owns and self._block is not None and self._pool is not None:
            self._pool.free(self._block)
        self._block = None
        self.t = None

    def _rebind(self, new_block):
        """Point this array at its block's new place after the pool was compacted."""
        shape, strides = tuple(self.t.shape), tuple(self.t.stride())
        n = self.t.numel()
        o = int(new_block) // 4
        self.t = self._pool.arena[o:o + max(n, 1)].as_strided(shape, strides)
        self._block = int(new_block)

    # -- swap state --------------------------------------------------------
    def is_swapout_ok(self):
        return self.gpu2cpu_event.query()

    def is_swapin_ok(self):
        if self.cpu2gpu_event.query():
            self.in_gpu = True
            return 1
        return 0

    def delete_itself(self):
        """Give the device bytes back but keep the object (shape, events)."""
        if self.in_gpu:
            self.in_gpu = False
            self._release()

    def malloc_itself(self):
        """Re-acquire device bytes for an array released by ``delete_itself``."""
        if self.t is None:
            fresh = empty(self._shape, self.ctx)
            self.t, self._block, self._pool = fresh.t, fresh._block, fresh._pool
            self._owns = True
            fresh._owns = False
            fresh._block = None
        self.in_gpu = True

    # -- micro tensors -----------------------------------------------------
    def split_tensor(self, total_number, dimension="batch"):
        """Create ``total_number`` views along batch (dim 0) or channel (dim 1),
        remainder spread over the first parts (reference:
        ``src/common/c_runtime_api.cc:212-271``).  Channel views are genuinely
        strided here; every kernel takes strides."""
        if self.split_number == total_number and self.split_dimension == dimension and self.sTensor:
            return self.sTensor
        self.splitted = True
        self.split_number = total_number
        self.split_dimension = dimension
        self.sTensor = [slice_for_micro_tensor(self, i, total_number, dimension)
                        for i in range(total_number)]
        return self.sTensor

    def merge(self):
        self.splitted = False
        self.sTensor = []
        self.split_number = 1
        self.in_gpu = True

    # -- copies --------------------------------------------------------------
    def numpy_view(self):
        """Zero-copy NumPy view (host-backed arrays only), logical indexing."""
        assert not self.is_cuda
        return self.t.numpy()

    def asnumpy(self):
        t = self.t
        if t.is_cuda:
            t = t.cpu()
        return np.ascontiguousarray(t.numpy()).astype(np.float32, copy=True)

    def _sync_copyfrom(self, source_array):
        if isinstance(source_array, NDArray):
            src = source_array.t
        else:
            src = torch.from_numpy(np.ascontiguousarray(source_array, dtype=np.float32))
        assert tuple(src.shape) == self._shape, "array shape do not match the shape of NDArray"
        self.t.copy_(src)
        return self

    def __setitem__(self, in_slice, value):
        if not isinstance(in_slice, slice) or in_slice.start is not None or in_slice.stop is not None:
            raise ValueError("Array only support set from numpy array")
        if isinstance(value, NDArray):
            if value is not self:
                value.copyto(self)
        elif isinstance(value, (np.ndarray, np.generic)):
            self._sync_copyfrom(value)
        else:
            raise TypeError("type %s not supported" % str(type(value)))

    def copyto(self, target, stream=None):
        """Copy into another NDArray or to a new array on a context."""
        if isinstance(target, DLContext):
            target = empty(self._shape, target)
        assert isinstance(target, NDArray)
        with _stream_scope(stream):
            target.t.copy_(self.t, non_blocking=stream is not None)
        return target

    def async_h2d(self, source, stream_handle=None, event_handle=None):
        """``self`` (device) <- ``source`` (pinned host), on ``stream_handle``."""
        with _stream_scope(stream_handle):
            self.t.copy_(source.t, non_blocking=True)
            if event_handle is not None:
                event_handle.record(stream_handle)

    def async_d2h(self, source, stream_handle=None, event_handle=None):
        """``self`` (pinned host) <- ``source`` (device), on ``stream_handle``."""
        with _stream_scope(stream_handle):
            self.t.copy_(source.t, non_blocking=True)
            if event_handle is not None:
                event_handle.record(stream_handle)


class _stream_scope(object):
    """Run torch copies on the framework stream (no-op for host contexts)."""

    def __init__(self, stream):
        self.ctxmgr = None
        if stream is not None and getattr(stream, "torch_stream", None) is not None:
            self.ctxmgr = torch.cuda.stream(stream.torch_stream)

    def __enter__(self):
        if self.ctxmgr is not None:
            self.ctxmgr.__enter__()

    def __exit__(self, *a):
        if self.ctxmgr is not None:
            self.ctxmgr.__exit__(*a)


def empty(shape, ctx=cpu(0), pinned=False, use_pool=True, channels_last=None, long_lived=False):
    """Uninitialised fp32 array on ``ctx``; goes through the context's pool when
    one is installed and raises :class:`OutOfHBMBudget` when it does not fit."""
    shape = tuple(int(s) for s in shape)
    n = _numel(shape)
    pool = _POOLS.get(ctx) if use_pool else None
    cl = is_cuda_ctx(ctx) if channels_last is None else (bool(channels_last) and is_cuda_ctx(ctx))
    if pool is not None:
        blk, view = pool.alloc_view(n * 4, shape, cl and len(shape) == 4, long_lived)
        return NDArray(view, ctx, block=blk, pool=pool)
    if ctx.device_type == 2:
        flat = torch.empty(max(n, 1), dtype=torch.float32, device=ctx.torch_device)
    else:
        flat = torch.empty(max(n, 1), dtype=torch.float32,
                           pin_memory=bool(pinned and torch.cuda.is_available()))
    return NDArray(_make_view(flat[:n], shape, cl), ctx)


def array(arr, ctx=cpu(0), use_pool=True, channels_last=None):
    """Create an array from a NumPy source (converted to fp32).  4-D arrays on a
    CUDA context are stored channels-last unless ``channels_last=False``."""
    arr = np.asarray(arr, dtype=np.float32)
    ret = empty(arr.shape, ctx, use_pool=use_pool, channels_last=channels_last)
    ret._sync_copyfrom(arr)
    return ret


def from_tensor(t, ctx):
    return NDArray(t, ctx)


def _split_bounds(extent, total, index):
    """[begin, end) of part ``index`` when ``extent`` is cut in ``total`` parts
    with the remainder given to the first parts."""
    base, rem = divmod(extent, total)
    begin = index * base + min(index, rem)
    return begin, begin + base + (1 if index < rem else 0)


def slice_for_micro_tensor(input_tensor, index, total_number, dimension="batch"):
    dim = {"batch": 0, "channel": 1}.get(dimension)
    if dim is None:
        raise NotImplementedError(dimension)
    b, e = _split_bounds(input_tensor.shape[dim], total_number, index)
    view = input_tensor.t.narrow(dim, b, e - b)
    out = NDArray(view, input_tensor.ctx, owns=False)
    out.in_gpu = True
    return out


def split_shape(input_shape, total_number=0, dimension="batch"):
    assert total_number > 0
    dim = {"batch": 0, "channel": 1}[dimension]
    shapes = []
    for i in range(total_number):
        b, e = _split_bounds(input_shape[dim], total_number, i)
        s = list(input_shape)
        s[dim] = e - b
        shapes.append(s)
    return shapes


def tensor_reuse(input_shape, output_shape, pieces, overlap_pieces, ctx=gpu(0)):
    """One buffer holding a micro-op's output at its head and the input at its
    tail, sized so that the last ``overlap_pieces`` output pieces may overwrite
    input pieces that were already consumed (reference:
    ``src/common/c_runtime_api.cc:164-210``).  Both arrays are row-major views
    (batch pieces are then contiguous byte ranges)."""
    n_in, n_out = _numel(input_shape), _numel(output_shape)
    in_piece = -(-n_in // pieces)
    total = n_out + in_piece * (pieces - overlap_pieces)
    total = max(total, n_in, n_out)
    holder = empty((total,), ctx)
    out = NDArray(holder.t[:n_out].view(tuple(output_shape)), ctx, owns=False)
    inp = NDArray(holder.t[total - n_in:].view(tuple(input_shape)), ctx, owns=False)
    out._holder = inp._holder = holder
    return inp, out


class ND_Sparse_Array(object):
    """CSR matrix (data, row offsets, column indices) on a context."""
    __slots__ = ["data", "row", "col", "nrow", "ncol", "ctx"]

    def __init__(self, data, row, col, nrow, ncol, ctx=None):
        self.data, self.row, self.col = data, row, col
        self.nrow, self.ncol, self.ctx = nrow, ncol, ctx

    @property
    def shape(self):
        return (self.nrow, self.ncol)

    def to_scipy(self):
        import scipy.sparse
        return scipy.sparse.csr_matrix(
            (self.data.asnumpy(), self.col.asnumpy().astype(np.int32),
             self.row.asnumpy().astype(np.int32)), shape=self.shape)


def sparse_array(values, indices, shape, ctx=cpu(0)):
    """COO triplets -> CSR arrays on ``ctx`` (reference ``ndarray.py:433-455``)."""
    import scipy.sparse
    mat = scipy.sparse.csr_matrix((values, (indices[0], indices[1])), shape=shape)
    return ND_Sparse_Array(array(mat.data, ctx), array(mat.indptr, ctx), array(mat.indices, ctx),
                           shape[0], shape[1], ctx)
