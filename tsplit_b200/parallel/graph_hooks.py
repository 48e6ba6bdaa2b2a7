"""In-graph gradient exchange (reference: the legacy ``Distributed_CommunicateOp``
and ``Ps_CommunicateOp`` nodes, ``python/athena/autodiff.py:233-340,810-862,917-954``).

``distributed_gradients(loss, vars, communicator)`` wraps every gradient in an
all-reduce node; ``ps_gradients(loss, vars, ps, lr)`` wraps it in a push / pull
node that pre-multiplies by ``-lr / num_workers`` so the servers accumulate the
weights, as the reference does (``autodiff.py:276-318``)."""
from __future__ import annotations

import numpy as np

from .. import ndarray
from ..graph import Op, gradients, phase_scope


class DistributedCommunicateOp(Op):
    name = "DistributedCommunicate"

    def __call__(self, g, communicator=None, average=True):
        return Op.__call__(self, g, communicator=communicator, average=average)

    def _world(self, comm):
        for attr in ("nRanks", "world", "devs_number"):
            if hasattr(comm, attr):
                return int(getattr(comm, attr))
        return 1

    def compute(self, node, input_vals, output_val, use_numpy=True, stream_handle=None):
        comm = node.attrs["communicator"]
        src = input_vals[0]
        if use_numpy:
            output_val[...] = src
            if comm is not None:
                comm.allReduce(output_val) if hasattr(comm, "allReduce") else comm.dlarrayNcclAllReduce(output_val)
                if node.attrs["average"]:
                    output_val /= self._world(comm)
            return
        from ..ops import _gpu as G
        G.copy(src, output_val, stream_handle)
        if comm is not None:
            if stream_handle is not None:
                stream_handle.sync()
            comm.dlarrayNcclAllReduce(output_val) if hasattr(comm, "dlarrayNcclAllReduce") else \
                comm.allReduce(output_val)
            if node.attrs["average"]:
                G.unary(G.UN_MULC, output_val, output_val, stream_handle, alpha=1.0 / self._world(comm))

    def gradient(self, node, g):
        raise NotImplementedError

    def infer_shape(self, node, s):
        return tuple(s[0])


class PsCommunicateOp(Op):
    name = "PsCommunicate"

    def __call__(self, g, var, ps=None, lr=0.01, mode="BSP"):
        return Op.__call__(self, g, var=var, ps=ps, lr=lr, mode=mode)

    def compute(self, node, input_vals, output_val, use_numpy=True, stream_handle=None):
        ps, var = node.attrs["ps"], node.attrs["var"]
        g = input_vals[0]
        if hasattr(ps, "push_pull_device") and not use_numpy and isinstance(g, ndarray.NDArray) and g.is_cuda:
            # GPU-resident shards: the push and the pull are one kernel over NVLink, nothing visits the host
            from ..ops import _gpu as G
            arr = ps.push_pull_device(var.name, g, node.attrs["lr"], node.attrs["mode"], stream_handle)
            G.copy(arr, output_val, stream_handle)
            var.tensor_value = arr               # the next forward pass reads the served value in place
            return
        g_np = g if isinstance(g, np.ndarray) else g.asnumpy()
        delta = (-node.attrs["lr"] / ps.num_workers) * g_np
        new_w = ps.push_pull(var.name, delta, mode=node.attrs["mode"])
        if isinstance(output_val, np.ndarray):
            output_val[...] = new_w.reshape(output_val.shape)
        else:
            output_val._sync_copyfrom(new_w.reshape(output_val.shape))
        tv = var.tensor_value
        if isinstance(tv, ndarray.NDArray):
            tv._sync_copyfrom(new_w.reshape(tv.shape))
        elif tv is not None:
            tv[...] = new_w.reshape(tv.shape)

    def gradient(self, node, g):
        raise NotImplementedError

    def infer_shape(self, node, s):
        return tuple(s[0])


_dist, _ps = DistributedCommunicateOp(), PsCommunicateOp()


def distributed_communicate_op(node, communicator=None, average=True):
    return _dist(node, communicator, average)


def ps_communicate_op(node, var, ps, lr=0.01, mode="BSP"):
    return _ps(node, var, ps, lr, mode)


def distributed_gradients(output_node, node_list, communicator=None, scheduler_policy=None):
    """Gradients followed by an all-reduce (average) node each."""
    grads = gradients(output_node, node_list)
    with phase_scope("backward"):
        return [distributed_communicate_op(g, communicator) for g in grads]


def ps_gradients(output_node, node_list, ps, lr=0.01, mode="BSP"):
    """Gradients pushed to the parameter servers; each returned node evaluates
    to the freshly pulled weight of its variable."""
    grads = gradients(output_node, node_list)
    if hasattr(ps, "push_pull_device"):          # GPU-resident shards: register the device values, then exchange handles
        for v in node_list:
            ps.init(v.name, v.tensor_value)
        ps.finalize()
        asp = mode == "ASP"
        for v in node_list:
            v.tensor_value = ps.value_array(v.name, asp=asp)
    else:
        for v in node_list:
            if v.tensor_value is not None:
                tv = v.tensor_value
                ps.init(v.name, tv.asnumpy() if isinstance(tv, ndarray.NDArray) else np.asarray(tv))
    with phase_scope("update"):
        return [ps_communicate_op(g, v, ps, lr, mode) for g, v in zip(grads, node_list)]
