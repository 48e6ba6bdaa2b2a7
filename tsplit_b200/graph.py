"""Define-then-run graph core: ``Node``, ``Op``, topological orders, ``gradients``.

Capability parity: ``python/athena/gpu_ops/Node.py:7-137`` and
``python/athena/gpu_ops/executor.py:160-332``.  Differences by design: op
attributes live on the node (``node.attrs``) instead of a fresh op instance per
call, and every node is tagged with the phase it was created in (``forward`` /
``backward`` / ``update``) at ``gradients()`` time, so executors do not have to
guess the phase boundary from the position of the first loss op.
"""
from __future__ import annotations

import itertools
from collections import deque

_node_ids = itertools.count()
_PHASE = ["forward"]
#: set by executors that run on a CPU context: operators use their native host kernels
CPU_NATIVE = [False]
#: operators of CPU-context executors that ran on NumPy because they have no native host kernel
NUMPY_FALLBACKS = [0]


class phase_scope(object):
    """Tag every node created inside the ``with`` block with ``name``."""

    def __init__(self, name):
        self.name = name

    def __enter__(self):
        self.prev = _PHASE[0]
        _PHASE[0] = self.name

    def __exit__(self, *a):
        _PHASE[0] = self.prev


class Node(object):
    """A value in the dataflow graph."""

    def __init__(self):
        self.inputs = []
        self.op = None
        self.const_attr = None
        self.name = ""
        self.desc = ""
        self.id = next(_node_ids)
        self.swap = False
        self.phase = _PHASE[0]
        self.attrs = {}
        self.profiler = None
        self.fwd_node = None      # for backward nodes: the forward node they differentiate

    def __add__(self, other):
        from .ops import elementwise as E
        if isinstance(other, Node):
            return E.add_op(self, other)
        return E.addbyconst_op(self, other)

    def __mul__(self, other):
        from .ops import elementwise as E
        if isinstance(other, Node):
            return E.mul_op(self, other)
        return E.mul_byconst_op(self, other)

    def __sub__(self, other):
        from .ops import elementwise as E
        if isinstance(other, Node):
            return E.add_op(self, E.opposite_op(other))
        return E.addbyconst_op(self, -other)

    def __neg__(self):
        from .ops import elementwise as E
        return E.opposite_op(self)

    __radd__ = __add__
    __rmul__ = __mul__

    def __str__(self):
        return self.name

    __repr__ = __str__

    def __lt__(self, other):
        return self.id < other.id


class Op(object):
    """Operation: builds nodes and knows how to compute / differentiate them.

    ``compute`` dispatches to ``np_compute`` (the NumPy oracle, also the CPU
    and simulated-GPU path) or ``gpu_compute`` (hand-written sm_100a kernels).
    """
    name = "Op"

    def __call__(self, *inputs, **attrs):
        node = Node()
        node.op = self
        node.inputs = list(inputs)
        node.attrs = attrs
        # names stay O(1): nesting the input names doubles their length at every join of a DAG
        node.name = self.name
        node.desc = "%s_%d" % (self.name, node.id)
        return node

    # -- execution ---------------------------------------------------------
    def compute(self, node, input_vals, output_val, use_numpy=True, stream_handle=None):
        if use_numpy:
            # executors on a CPU context (ndarray.cpu) route the operators that have one through the native
            # host library (cpu_links -> csrc/runtime/cpu_ops.cc); ctx=None stays pure NumPy, the oracle
            if CPU_NATIVE[0] and output_val is not None and self.cpu_compute(node, input_vals, output_val):
                return output_val
            if CPU_NATIVE[0]:
                NUMPY_FALLBACKS[0] += 1          # a CPU-context step with one of these cannot be replayed natively
            res = self.np_compute(node, input_vals)
            if output_val is not None and res is not None:
                output_val[...] = res
            return res
        return self.gpu_compute(node, input_vals, output_val, stream_handle)

    def np_compute(self, node, input_vals):
        raise NotImplementedError(self.name)

    def cpu_compute(self, node, input_vals, output_val):
        """Native host kernel (OpenMP) writing ``output_val``; returns False when the op has none or the
        operands do not qualify (then the NumPy path runs)."""
        return False

    def gpu_compute(self, node, input_vals, output_val, stream_handle):
        raise NotImplementedError("%s has no GPU kernel" % self.name)

    def gradient(self, node, output_grad):
        raise NotImplementedError(self.name)

    def infer_shape(self, node, input_shapes):
        raise NotImplementedError(self.name)

    # -- cost model hooks (see profiler.py) -----------------------------------
    def flops(self, node, input_shapes, output_shape):
        """Floating point operations of one execution (default: 1 per output)."""
        n = 1
        for s in output_shape or ():
            n *= s
        return float(n)

    def workspace_bytes(self, node, input_shapes, output_shape):
        return 0

    # True when the op only re-views / copies data and is cheap to recompute
    cheap = False


# -----------------------------------------------------------------------------
def find_topo_sort(node_list):
    """Post-order DFS (iterative; graphs here reach thousands of nodes)."""
    visited, order = set(), []
    for root in node_list:
        if root in visited:
            continue
        stack = [(root, iter(root.inputs))]
        visited.add(root)
        while stack:
            node, it = stack[-1]
            advanced = False
            for child in it:
                if child not in visited:
                    visited.add(child)
                    stack.append((child, iter(child.inputs)))
                    advanced = True
                    break
            if not advanced:
                order.append(node)
                stack.pop()
    return order


def find_topo_sort2(node_list):
    """Kahn order with a FIFO frontier (O(N + E)); ties resolved by creation
    id, so forward nodes precede the backward nodes created after them."""
    nodes = find_topo_sort(node_list)
    indeg = {n: 0 for n in nodes}
    users = {n: [] for n in nodes}
    for n in nodes:
        for i in set(n.inputs):
            indeg[n] += 1
            users[i].append(n)
    ready = deque(sorted(n for n in nodes if indeg[n] == 0))
    order = []
    while ready:
        n = ready.popleft()
        order.append(n)
        for u in sorted(users[n]):
            indeg[u] -= 1
            if indeg[u] == 0:
                ready.append(u)
    assert len(order) == len(nodes), "graph has a cycle"
    return order


def schedule_order(node_list):
    """Execution order used by every executor: dependency order with creation
    id as the priority.  Creation order interleaves each data gradient with its
    filter gradient exactly as back-propagation produced them, which keeps
    activation lifetimes short."""
    import heapq
    nodes = find_topo_sort(node_list)
    indeg = {n: len(set(n.inputs)) for n in nodes}
    users = {n: [] for n in nodes}
    for n in nodes:
        for i in set(n.inputs):
            users[i].append(n)
    heap = [(n.id, n) for n in nodes if indeg[n] == 0]
    heapq.heapify(heap)
    order = []
    while heap:
        _, n = heapq.heappop(heap)
        order.append(n)
        for u in users[n]:
            indeg[u] -= 1
            if indeg[u] == 0:
                heapq.heappush(heap, (u.id, u))
    return order


def sum_node_list(node_list):
    """Sum of the non-None nodes (None when there is none)."""
    from .ops import elementwise as E
    parts = [n for n in node_list if n is not None]
    if not parts:
        return None
    acc = parts[0]
    for p in parts[1:]:
        acc = E.add_op(acc, p)
    return acc


def gradients(output_node, node_list):
    """Reverse-mode autodiff: adjoint nodes of ``output_node`` w.r.t. ``node_list``.

    Nodes that do not influence the output are dropped from the result (as in
    the reference, ``executor.py:195``)."""
    from .ops.misc import oneslike_op
    with phase_scope("backward"):
        adj = {output_node: [oneslike_op(output_node)]}
        node_to_grad = {}
        for node in reversed(find_topo_sort([output_node])):
            g = sum_node_list(adj.get(node, []))
            if g is None:
                continue
            node_to_grad[node] = g
            if not node.inputs:
                continue
            in_grads = node.op.gradient(node, g)
            if in_grads is None:
                continue
            for inp, ig in zip(node.inputs, in_grads):
                if ig is not None:
                    if ig.fwd_node is None:
                        ig.fwd_node = node
                    adj.setdefault(inp, []).append(ig)
    return [node_to_grad[n] for n in node_list if n in node_to_grad]


def broadcast_rule(shape_a, shape_b):
    """NumPy broadcasting of two shapes."""
    a, b = list(shape_a), list(shape_b)
    if len(a) < len(b):
        a = [1] * (len(b) - len(a)) + a
    else:
        b = [1] * (len(a) - len(b)) + b
    out = []
    for x, y in zip(a, b):
        assert x == y or x == 1 or y == 1, "shapes %s and %s do not broadcast" % (shape_a, shape_b)
        out.append(max(x, y))
    return tuple(out)
