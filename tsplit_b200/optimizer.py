"""Optimizers: SGD, Momentum (optionally Nesterov), AdaGrad, Adam.

Capability parity: ``python/athena/optimizer.py:8-290`` — ``get_var_list``,
``initiate_vars``, ``minimize`` (= ``gradients`` + an in-graph ``OptimizerOp``),
same constructor defaults and update formulas (``src/ops/Optimizers.cu:3-149``).

GPU path: one multi-tensor launch covers up to 64 parameter tensors (pointer
table in kernel parameters) instead of one launch per parameter.  When a
data-parallel communicator is attached (``parallel/ddp.py``) the update is done
by the fused all-reduce kernel and this path is skipped.
"""
from __future__ import annotations

import numpy as np

from . import ndarray
from .graph import Op, find_topo_sort, gradients, phase_scope
from .ops import _gpu as G
from .ops.misc import PlaceholderOp


class Optimizer(object):
    """Base optimizer."""
    name = "Optimizer"
    kind = 0

    def __init__(self, ctx=None):
        self.tensors = None
        self.ctx = ctx
        self.initiated = False
        self.step_count = 0
        self.communicator = None      # set by parallel.ddp to fuse all-reduce + update

    @property
    def params(self):
        """Current values of the optimised variables (resolved on every use: an
        executor may have moved a NumPy initial value onto its device)."""
        return [n.tensor_value for n in self.tensors]

    @staticmethod
    def get_var_list(loss):
        def trainable(n):
            return isinstance(n.op, PlaceholderOp) and getattr(n, "trainable", False)
        return [n for n in find_topo_sort([loss]) if trainable(n)]

    def initiate_states(self):
        pass

    def _zeros_like_params(self, value=0.0):
        if ndarray.is_gpu_ctx(self.ctx):
            out = []
            for p in self.params:
                a = ndarray.empty(p.shape, self.ctx, use_pool=False)
                a.t.fill_(value)
                out.append(a)
            return out
        return [np.full(p.shape, value, dtype=np.float32) for p in self.params]

    def initiate_vars(self):
        """Move every variable's value to the optimizer's context."""
        for node in self.tensors:
            v = node.tensor_value
            if ndarray.is_gpu_ctx(self.ctx):
                if isinstance(v, np.ndarray):
                    node.tensor_value = ndarray.array(v, self.ctx, use_pool=False)
                elif isinstance(v, ndarray.NDArray) and v.ctx != self.ctx:
                    node.tensor_value = ndarray.array(v.asnumpy(), self.ctx, use_pool=False)
            elif isinstance(v, ndarray.NDArray):
                node.tensor_value = v.asnumpy()
            else:
                node.tensor_value = np.ascontiguousarray(v, dtype=np.float32)
        self.initiate_states()
        self.initiated = True

    def minimize(self, loss, var_list=None):
        self.loss = loss
        if not var_list:
            var_list = self.get_var_list(loss)
        self.tensors = list(var_list)
        grads = gradients(loss, self.tensors)
        assert len(grads) == len(self.tensors), "some variables do not influence the loss"
        self.initiate_vars()
        with phase_scope("update"):
            return _optimizer_op(grads, self)

    # -- update ---------------------------------------------------------------
    def hyper(self):
        return []

    def slots(self):
        return None, None

    def update(self, grads, use_numpy=False, stream_handle=None):
        assert self.initiated is True
        assert len(grads) == len(self.params)
        self.step_count += 1
        self._begin_step()
        if self.communicator is not None:
            self.communicator.reduce_and_update(self, grads, stream_handle)
            return
        on_device = ndarray.is_gpu_ctx(self.ctx) and self.ctx.device_type == 2
        params = self.params
        if on_device and not use_numpy:
            s1, s2 = self.slots()
            hdev = self._device_hyper(stream_handle)
            for lo in range(0, len(grads), 64):
                hi = lo + 64
                G.optimizer_step(self.kind, params[lo:hi], grads[lo:hi],
                                 s1[lo:hi] if s1 else None, s2[lo:hi] if s2 else None,
                                 self.hyper(), stream_handle, hyper_dev=hdev)
            return
        from . import graph, cpu_links
        native = graph.CPU_NATIVE[0]          # an executor on ndarray.cpu: the OpenMP update kernels
        s1, s2 = self.slots() if native else (None, None)
        for i, g in enumerate(grads):
            p = params[i]
            pv = p.numpy_view() if isinstance(p, ndarray.NDArray) else p
            gv = g.numpy_view() if isinstance(g, ndarray.NDArray) else g
            if native:
                a = self._np(s1[i]) if s1 else None
                b = self._np(s2[i]) if s2 else None
                if cpu_links.ok(pv, gv, *[x for x in (a, b) if x is not None]) and pv.shape == gv.shape:
                    cpu_links.optimizer_update(self.kind, pv, gv, a, b, self.hyper())
                    if self.kind == 4:
                        from .runtime import tape
                        if tape.ACTIVE[0] is not None:      # the bias-correction powers are part of the recorded bytes
                            tape.ACTIVE[0].invalid = "Adam's hyper-parameters change every step"
                    continue
                graph.NUMPY_FALLBACKS[0] += 1
            self._np_update(i, pv, gv)

    def _begin_step(self):
        pass

    def _device_hyper(self, stream):
        """Device-resident per-step scalars of the update kernel (Adam); None otherwise."""
        return None

    def _np(self, arr):
        return arr.numpy_view() if isinstance(arr, ndarray.NDArray) else arr

    # -- checkpointing of optimizer state (extra keys old loaders ignore) -----------
    def state_dict(self):
        out = {"__step__": self.step_count}
        s1, s2 = self.slots()
        for node, a, b in zip(self.tensors, s1 or [None] * len(self.tensors), s2 or [None] * len(self.tensors)):
            for slot, arr in (("slot1", a), ("slot2", b)):
                if arr is not None:
                    out["__optimizer__/%s/%s" % (node.name, slot)] = (
                        arr.asnumpy() if isinstance(arr, ndarray.NDArray) else np.array(arr))
        return out

    def load_state_dict(self, state):
        self.step_count = int(state.get("__step__", 0))
        s1, s2 = self.slots()
        for node, a, b in zip(self.tensors, s1 or [None] * len(self.tensors), s2 or [None] * len(self.tensors)):
            for slot, arr in (("slot1", a), ("slot2", b)):
                key = "__optimizer__/%s/%s" % (node.name, slot)
                if arr is not None and key in state:
                    if isinstance(arr, ndarray.NDArray):
                        arr._sync_copyfrom(np.asarray(state[key], dtype=np.float32))
                    else:
                        arr[...] = state[key]
        self._restore_step()

    def _restore_step(self):
        pass


class OptimizerOp(Op):
    name = "Optimizer"

    def __call__(self, grads, optimizer):
        node = Op.__call__(self, *grads)
        node.attrs["optimizer"] = optimizer
        node.name = "Optimizer_%s" % optimizer.name
        return node

    def compute(self, node, input_vals, output_val, use_numpy=True, stream_handle=None):
        assert output_val is None
        node.attrs["optimizer"].update(input_vals, use_numpy, stream_handle)

    def gradient(self, node, g):
        raise NotImplementedError

    def infer_shape(self, node, s):
        return None


_optimizer_op_inst = OptimizerOp()


def _optimizer_op(grads, optimizer):
    return _optimizer_op_inst(grads, optimizer)


class SGDOptimizer(Optimizer):
    name, kind = "SGD", 0

    def __init__(self, learning_rate=0.01, ctx=None):
        super(SGDOptimizer, self).__init__(ctx)
        self.learning_rate = learning_rate

    def hyper(self):
        return [self.learning_rate]

    def _np_update(self, i, p, g):
        p[...] = p - self.learning_rate * g


class MomentumOptimizer(Optimizer):
    name = "Momentum"

    def __init__(self, learning_rate=0.01, momentum=0.9, nesterov=False, ctx=None):
        super(MomentumOptimizer, self).__init__(ctx)
        self.learning_rate, self.momentum, self.nesterov = learning_rate, momentum, nesterov
        self.kind = 2 if nesterov else 1

    def initiate_states(self):
        self.velocity = self._zeros_like_params()

    def hyper(self):
        return [self.learning_rate, self.momentum]

    def slots(self):
        return self.velocity, None

    def _np_update(self, i, p, g):
        v = self._np(self.velocity[i])
        if self.nesterov:
            lr_g = -self.learning_rate * g
            v[...] = self.momentum * (v + lr_g)
            p[...] = p + v + lr_g
        else:
            v[...] = self.momentum * v - self.learning_rate * g
            p[...] = p + v


class AdaGradOptimizer(Optimizer):
    name, kind = "AdaGrad", 3

    def __init__(self, learning_rate=0.01, initial_accumulator_value=0.0, eps=1e-7, ctx=None):
        assert learning_rate >= 0, "learning rate must be non-negative"
        assert initial_accumulator_value >= 0.0, "initial accumulator value must be non-negative"
        assert eps > 0.0, "epsilon must be positive"
        super(AdaGradOptimizer, self).__init__(ctx)
        self.learning_rate, self.initial_accumulator_value, self.eps = (
            learning_rate, initial_accumulator_value, eps)

    def initiate_states(self):
        self.accumulator_value = self._zeros_like_params(self.initial_accumulator_value)

    def hyper(self):
        return [self.learning_rate, self.eps]

    def slots(self):
        return self.accumulator_value, None

    def _np_update(self, i, p, g):
        acc = self._np(self.accumulator_value[i])
        acc[...] = acc + g * g
        p[...] = p - self.learning_rate * g / (np.sqrt(acc) + self.eps)


class AdamOptimizer(Optimizer):
    name, kind = "Adam", 4

    def __init__(self, learning_rate=0.01, beta1=0.9, beta2=0.999, epsilon=1e-7, ctx=None):
        super(AdamOptimizer, self).__init__(ctx)
        self.learning_rate, self.beta1, self.beta2, self.epsilon = learning_rate, beta1, beta2, epsilon
        self.beta1_t = 1.0
        self.beta2_t = 1.0

    def initiate_states(self):
        self.m = self._zeros_like_params()
        self.v = self._zeros_like_params()

    def _begin_step(self):
        self.beta1_t *= self.beta1
        self.beta2_t *= self.beta2

    def _restore_step(self):
        self.beta1_t = self.beta1 ** self.step_count
        self.beta2_t = self.beta2 ** self.step_count
        self._bt_dev = None                  # rebuilt from the restored powers on the next device step

    def _device_hyper(self, stream):
        """{beta1^t, beta2^t} on the device, advanced by a one-thread kernel every step, so that a step
        captured in a CUDA graph keeps the right bias correction when it is replayed."""
        bt = getattr(self, "_bt_dev", None)
        if bt is None:
            prev1 = self.beta1_t / self.beta1      # _begin_step already advanced the host copies
            prev2 = self.beta2_t / self.beta2
            bt = self._bt_dev = ndarray.array(np.array([prev1, prev2], np.float32), self.ctx, use_pool=False)
        G.adam_advance(bt, self.beta1, self.beta2, stream)
        return bt

    def hyper(self):
        return [self.learning_rate, self.beta1, self.beta2, self.beta1_t, self.beta2_t, self.epsilon]

    def slots(self):
        return self.m, self.v

    def _np_update(self, i, p, g):
        m, v = self._np(self.m[i]), self._np(self.v[i])
        m[...] = self.beta1 * m + (1 - self.beta1) * g
        v[...] = self.beta2 * v + (1 - self.beta2) * g * g
        mc = m / (1 - self.beta1_t)
        vc = v / (1 - self.beta2_t)
        p[...] = p - self.learning_rate * mc / (np.sqrt(vc) + self.epsilon)
