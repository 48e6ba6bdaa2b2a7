"""Element-wise op family.

Capability parity with the reference's ``gpu_ops/AddElewise.py:55-112``,
``AddConst.py:45-67``, ``MultiplyElewise.py:56-112``, ``MultiplyConst.py:45-69``,
``Division.py:41-133``, ``Opposite.py``, ``Sqrt.py:58-126``, ``Sigmoid.py``,
``Tanh.py``, ``Relu.py:31-104`` and ``Where.py:35-62``.

GPU path: one vectorised kernel per arity (``csrc/kernels/elementwise.cu``); the
"one side has shape (1,)" case reads the scalar on the device instead of the
reference's blocking ``.asnumpy()[0]`` host read (``AddElewise.py:86-93``).
"""
from __future__ import annotations

import numpy as np

from ..graph import Op
from . import _gpu as G


def _is_scalar_shape(s):
    return tuple(s) == (1,)


class _Binary(Op):
    gpu_code = 0

    def __call__(self, a, b):
        return Op.__call__(self, a, b)

    def _np(self, a, b):
        raise NotImplementedError

    def np_compute(self, node, iv):
        return self._np(iv[0], iv[1])

    def cpu_compute(self, node, iv, out):
        from .. import cpu_links
        code = cpu_links.BINARY.get(self.name)
        if code is None or not cpu_links.ok(iv[0], iv[1], out) or iv[0].shape != out.shape or iv[1].shape != out.shape:
            return False
        cpu_links.binary(code, iv[0], iv[1], out)
        return True

    def gpu_compute(self, node, iv, out, stream):
        a, b = iv
        if _is_scalar_shape(a.shape) and not _is_scalar_shape(b.shape):
            G.binary_dev_scalar(self.gpu_code, b, a, out, stream, scalar_first=True)
        elif _is_scalar_shape(b.shape) and not _is_scalar_shape(a.shape):
            G.binary_dev_scalar(self.gpu_code, a, b, out, stream, scalar_first=False)
        else:
            G.binary(self.gpu_code, a, b, out, stream)

    def infer_shape(self, node, s):
        if tuple(s[0]) == tuple(s[1]):
            return tuple(s[0])
        if _is_scalar_shape(s[0]):
            return tuple(s[1])
        if _is_scalar_shape(s[1]):
            return tuple(s[0])
        raise AssertionError("%s: shapes %s / %s differ" % (self.name, s[0], s[1]))


class AddOp(_Binary):
    name, gpu_code, cheap = "Add", G.BIN_ADD, True

    def _np(self, a, b):
        return a + b

    def gradient(self, node, g):
        return [g, g]


class MulOp(_Binary):
    name, gpu_code, cheap = "Mul", G.BIN_MUL, True

    def _np(self, a, b):
        return a * b

    def gradient(self, node, g):
        return [mul_op(node.inputs[1], g), mul_op(node.inputs[0], g)]


class DivOp(_Binary):
    name, gpu_code, cheap = "Div", G.BIN_DIV, True

    def _np(self, a, b):
        return a / b

    def gradient(self, node, g):
        a, b = node.inputs
        inv_b = div_const_op(1.0, b)
        return [mul_op(inv_b, g), mul_op(opposite_op(mul_op(div_op(a, b), inv_b)), g)]


class ReluGradientOp(_Binary):
    """``(sign(x)+1)/2 * g`` — note that x == 0 passes half the gradient, as the
    reference kernel does (``src/ops/Relu.cu:73-80``)."""
    name, gpu_code, cheap = "ReluGradient", G.BIN_RELU_GRAD, True

    def _np(self, x, g):
        return (np.sign(x) + 1) * 0.5 * g

    def gradient(self, node, g):
        raise NotImplementedError("second-order gradient of relu")


class AddReluOp(_Binary):
    """``relu(a + b)`` in one pass (the residual join of a ResNet block).  No counterpart in the
    reference, which runs ``AddOp`` then ``ReluOp`` (``examples/imagenet_resnet.py``): two extra passes
    over the tensor forward, and a backward that needs the pre-activation.  Here the backward masks
    by the OUTPUT (positive output = positive pre-activation) and both inputs share one gradient node."""
    name, gpu_code, cheap = "AddRelu", G.BIN_ADD_RELU, True

    def _np(self, a, b):
        return np.maximum(a + b, 0)

    def gradient(self, node, g):
        r = relu_out_gradient_op(node, g)
        return [r, r]


class ReluOutGradientOp(_Binary):
    """``g`` where the ReLU output ``y`` is positive, else 0."""
    name, gpu_code, cheap = "ReluOutGradient", G.BIN_RELU_GRAD_OUT, True

    def _np(self, y, g):
        return np.where(y > 0, g, 0).astype(np.float32)

    def gradient(self, node, g):
        raise NotImplementedError("second-order gradient of relu")


class _Unary(Op):
    gpu_code = 0
    cheap = True

    def __call__(self, x, const=None):
        node = Op.__call__(self, x)
        node.const_attr = const
        return node

    def np_compute(self, node, iv):
        return self._np(iv[0], node.const_attr)

    def cpu_compute(self, node, iv, out):
        from .. import cpu_links
        code = cpu_links.UNARY.get(self.name)
        if code is None or not cpu_links.ok(iv[0], out) or iv[0].shape != out.shape:
            return False
        cpu_links.unary(code, iv[0], out, 0.0 if node.const_attr is None else float(node.const_attr))
        return True

    def gpu_compute(self, node, iv, out, stream):
        G.unary(self.gpu_code, iv[0], out, stream,
                alpha=0.0 if node.const_attr is None else float(node.const_attr))

    def infer_shape(self, node, s):
        return tuple(s[0])


class AddConstOp(_Unary):
    name, gpu_code = "AddConst", G.UN_ADDC

    def _np(self, x, c):
        return x + c

    def gradient(self, node, g):
        return [g]


class MulConstOp(_Unary):
    name, gpu_code = "MulConst", G.UN_MULC

    def _np(self, x, c):
        return x * c

    def gradient(self, node, g):
        return [mul_byconst_op(g, node.const_attr)]


class DivConstOp(_Unary):
    """``c / x``."""
    name, gpu_code = "DivConst", G.UN_CDIV

    def _np(self, x, c):
        return c / x

    def gradient(self, node, g):
        x = node.inputs[0]
        # d(c/x) = -c/x^2
        return [mul_op(mul_byconst_op(mul_op(div_const_op(1.0, x), div_const_op(1.0, x)),
                                      -node.const_attr), g)]


class OppositeOp(_Unary):
    name, gpu_code = "Opposite", G.UN_NEG

    def _np(self, x, c):
        return -x

    def gradient(self, node, g):
        return [opposite_op(g)]


class SqrtOp(_Unary):
    name, gpu_code = "Sqrt", G.UN_SQRT

    def _np(self, x, c):
        return np.sqrt(x)

    def gradient(self, node, g):
        return [mul_op(mul_byconst_op(rsqrt_op(node.inputs[0]), 0.5), g)]


class RsqrtOp(_Unary):
    name, gpu_code = "Rsqrt", G.UN_RSQRT

    def _np(self, x, c):
        return 1.0 / np.sqrt(x)

    def gradient(self, node, g):
        x = node.inputs[0]
        return [mul_op(mul_byconst_op(div_op(rsqrt_op(x), x), -0.5), g)]


class SigmoidOp(_Unary):
    name, gpu_code = "Sigmoid", G.UN_SIGMOID

    def _np(self, x, c):
        return 1.0 / (1.0 + np.exp(-x))

    def gradient(self, node, g):
        # s * (1 - s)
        one_minus = addbyconst_op(opposite_op(node), 1.0)
        return [mul_op(mul_op(node, one_minus), g)]


class TanhOp(_Unary):
    name, gpu_code = "Tanh", G.UN_TANH

    def _np(self, x, c):
        return np.tanh(x)

    def gradient(self, node, g):
        return [mul_op(addbyconst_op(opposite_op(mul_op(node, node)), 1.0), g)]


class ReluOp(_Unary):
    name, gpu_code = "Relu", G.UN_RELU

    def _np(self, x, c):
        return np.maximum(x, 0)

    def gradient(self, node, g):
        return [relu_gradient_op(node.inputs[0], g)]


class WhereOp(Op):
    name, cheap = "Where", True

    def __call__(self, cond, a, b):
        return Op.__call__(self, cond, a, b)

    def np_compute(self, node, iv):
        return np.where(iv[0] != 0, iv[1], iv[2])

    def gpu_compute(self, node, iv, out, stream):
        G.where(iv[0], iv[1], iv[2], out, stream)

    def gradient(self, node, g):
        from .misc import zeroslike_op
        z = zeroslike_op(g)
        c = node.inputs[0]
        return [None, where_op(c, g, z), where_op(c, z, g)]

    def infer_shape(self, node, s):
        assert tuple(s[0]) == tuple(s[1]) == tuple(s[2])
        return tuple(s[0])


_add, _mul, _div, _relu_grad = AddOp(), MulOp(), DivOp(), ReluGradientOp()
_add_relu, _relu_out_grad = AddReluOp(), ReluOutGradientOp()
_addc, _mulc, _divc = AddConstOp(), MulConstOp(), DivConstOp()
_neg, _sqrt, _rsqrt, _sig, _tanh, _relu, _where = (OppositeOp(), SqrtOp(), RsqrtOp(), SigmoidOp(),
                                                   TanhOp(), ReluOp(), WhereOp())


def add_op(node_A, node_B):
    # x + broadcasttoTF_op(b, x): one kernel that reads b through broadcast strides
    for x, bc in ((node_A, node_B), (node_B, node_A)):
        if bc.op.name == "BroadcastToTF" and bc.inputs[1] is x and x.op.name != "BroadcastToTF":
            from .shape import add_broadcast_op
            return add_broadcast_op(x, bc.inputs[0])
    return _add(node_A, node_B)


def addbyconst_op(node, const_val):
    return _addc(node, const_val)


def mul_op(node_A, node_B):
    return _mul(node_A, node_B)


def mul_byconst_op(node, const_val):
    return _mulc(node, const_val)


def div_op(node_A, node_B):
    return _div(node_A, node_B)


def div_const_op(const_val, node_A):
    return _divc(node_A, const_val)


def opposite_op(node):
    return _neg(node)


def sqrt_op(node):
    return _sqrt(node)


def rsqrt_op(node):
    return _rsqrt(node)


def sigmoid_op(node):
    return _sig(node)


def tanh_op(node):
    return _tanh(node)


def relu_op(node):
    return _relu(node)


def relu_gradient_op(node, grad_node):
    return _relu_grad(node, grad_node)


def add_relu_op(node_A, node_B):
    return _add_relu(node_A, node_B)


def relu_out_gradient_op(out_node, grad_node):
    return _relu_out_grad(out_node, grad_node)


def where_op(cond, node_A, node_B):
    return _where(cond, node_A, node_B)
