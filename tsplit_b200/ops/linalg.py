"""Matrix products: dense 2-D, batched N-D and CSR-sparse x dense.

Capability parity: ``gpu_ops/MatrixMult.py:57-137``, ``BatchMatrixMult.py:49-130``,
``CuSparse.py:49-222`` (cuBLAS ``Sgemm`` / ``SgemmStridedBatched`` and legacy
cuSPARSE in ``src/ops/MatrixMult.cu``, ``BatchMatrixMult.cu``, ``CuSparseCsrmm.cu``).

GPU path: one TF32 tcgen05 kernel (TMA-fed, TMEM accumulators) handles all four
transpose combinations through K-major / MN-major shared-memory descriptors, so
no operand is ever transposed in memory; the batch is a grid dimension.
"""
from __future__ import annotations

import numpy as np

from ..graph import Op
from . import _gpu as G


def _mm_shape(sa, sb, ta, tb):
    m, k = (sa[-1], sa[-2]) if ta else (sa[-2], sa[-1])
    k2, n = (sb[-1], sb[-2]) if tb else (sb[-2], sb[-1])
    assert k == k2, "matmul inner dims differ: %s %s" % (sa, sb)
    return m, n, k


class MatMulOp(Op):
    name = "MatMul"

    def __call__(self, a, b, trans_A=False, trans_B=False):
        return Op.__call__(self, a, b, trans_A=trans_A, trans_B=trans_B)

    def np_compute(self, node, iv):
        a, b = iv
        a = a.T if node.attrs["trans_A"] else a
        b = b.T if node.attrs["trans_B"] else b
        return np.matmul(a, b)

    def cpu_compute(self, node, iv, out):
        from .. import cpu_links
        a, b = iv
        if not (cpu_links.ok(a, b, out) and a.ndim == 2 and b.ndim == 2):
            return False
        cpu_links.matrix_multiply(a, b, out, node.attrs["trans_A"], node.attrs["trans_B"])
        return True

    def gpu_compute(self, node, iv, out, stream):
        a, b = iv
        ta, tb = node.attrs["trans_A"], node.attrs["trans_B"]
        m, n, k = _mm_shape(a.shape, b.shape, ta, tb)
        assert a.is_contiguous() and b.is_contiguous() and out.is_contiguous()
        G.gemm(a, b, out, ta, tb, stream, m=m, n=n, k=k,
               lda=a.shape[1], ldb=b.shape[1], ldc=out.shape[1])

    def gradient(self, node, g):
        a, b = node.inputs
        ta, tb = node.attrs["trans_A"], node.attrs["trans_B"]
        if not ta and not tb:        # C = A B
            return [matmul_op(g, b, False, True), matmul_op(a, g, True, False)]
        if ta and not tb:            # C = A^T B
            return [matmul_op(b, g, False, True), matmul_op(a, g, False, False)]
        if not ta and tb:            # C = A B^T
            return [matmul_op(g, b, False, False), matmul_op(g, a, True, False)]
        return [matmul_op(b, g, True, True), matmul_op(g, a, True, True)]   # C = A^T B^T

    def infer_shape(self, node, s):
        m, n, _ = _mm_shape(s[0], s[1], node.attrs["trans_A"], node.attrs["trans_B"])
        return (m, n)

    def flops(self, node, s, out):
        m, n, k = _mm_shape(s[0], s[1], node.attrs["trans_A"], node.attrs["trans_B"])
        return 2.0 * m * n * k


class BatchMatMulOp(Op):
    name = "BatchMatMul"

    def __call__(self, a, b, trans_A=False, trans_B=False):
        return Op.__call__(self, a, b, trans_A=trans_A, trans_B=trans_B)

    def np_compute(self, node, iv):
        a, b = iv
        if node.attrs["trans_A"]:
            a = np.swapaxes(a, -1, -2)
        if node.attrs["trans_B"]:
            b = np.swapaxes(b, -1, -2)
        return np.matmul(a, b)

    def gpu_compute(self, node, iv, out, stream):
        a, b = iv
        ta, tb = node.attrs["trans_A"], node.attrs["trans_B"]
        m, n, k = _mm_shape(a.shape, b.shape, ta, tb)
        batch = 1
        for d in a.shape[:-2]:
            batch *= d
        assert a.is_contiguous() and b.is_contiguous() and out.is_contiguous()
        G.gemm(a, b, out, ta, tb, stream, batch=batch, m=m, n=n, k=k,
               sa=a.shape[-1] * a.shape[-2], sb=b.shape[-1] * b.shape[-2], sc=m * n,
               lda=a.shape[-1], ldb=b.shape[-1], ldc=n)

    def gradient(self, node, g):
        a, b = node.inputs
        ta, tb = node.attrs["trans_A"], node.attrs["trans_B"]
        if not ta and not tb:
            return [batch_matmul_op(g, b, False, True), batch_matmul_op(a, g, True, False)]
        if ta and not tb:
            return [batch_matmul_op(b, g, False, True), batch_matmul_op(a, g, False, False)]
        if not ta and tb:
            return [batch_matmul_op(g, b, False, False), batch_matmul_op(g, a, True, False)]
        return [batch_matmul_op(b, g, True, True), batch_matmul_op(g, a, True, True)]

    def infer_shape(self, node, s):
        assert tuple(s[0][:-2]) == tuple(s[1][:-2]), "batch dims differ"
        m, n, _ = _mm_shape(s[0], s[1], node.attrs["trans_A"], node.attrs["trans_B"])
        return tuple(s[0][:-2]) + (m, n)

    def flops(self, node, s, out):
        m, n, k = _mm_shape(s[0], s[1], node.attrs["trans_A"], node.attrs["trans_B"])
        b = 1
        for d in s[0][:-2]:
            b *= d
        return 2.0 * b * m * n * k


class CsrmmOp(Op):
    """``op(A_csr) · op(B)``; the sparse matrix is a constant attribute of the
    node's first input (a placeholder fed with an ``ND_Sparse_Array``)."""
    name = "Csrmm"

    def __call__(self, a, b, trans_A=False, trans_B=False, vector=False):
        return Op.__call__(self, a, b, trans_A=trans_A, trans_B=trans_B, vector=vector)

    def _dense_b(self, node, b):
        return b

    def np_compute(self, node, iv):
        a, b = iv
        mat = a if not hasattr(a, "to_scipy") else a.to_scipy()
        if node.attrs["trans_A"]:
            mat = mat.T
        bb = b.T if node.attrs["trans_B"] else b
        res = mat @ bb
        return np.asarray(res, dtype=np.float32)

    def gpu_compute(self, node, iv, out, stream):
        a, b = iv
        assert not node.attrs["trans_B"], "csrmm: trans_B is not supported on the GPU path"
        ncols = 1 if node.attrs["vector"] else b.shape[1]
        G.csrmm(a.data, a.row, a.col, a.nrow, a.ncol, b, out, node.attrs["trans_A"], ncols, stream)

    def gradient(self, node, g):
        a, b = node.inputs
        at = node.attrs
        if at["vector"]:
            return [None, csrmv_op(a, g, not at["trans_A"])]
        gb = csrmm_op(a, g, not at["trans_A"], False)
        if at["trans_B"]:
            from .shape import transpose_op
            gb = transpose_op(gb)
        return [None, gb]

    def infer_shape(self, node, s):
        at = node.attrs
        rows = s[0][1] if at["trans_A"] else s[0][0]
        if at["vector"]:
            return (rows,)
        cols = s[1][0] if at["trans_B"] else s[1][1]
        return (rows, cols)


_mm, _bmm, _csr = MatMulOp(), BatchMatMulOp(), CsrmmOp()


def matmul_op(node_A, node_B, trans_A=False, trans_B=False):
    return _mm(node_A, node_B, trans_A, trans_B)


def batch_matmul_op(node_A, node_B, trans_A=False, trans_B=False):
    return _bmm(node_A, node_B, trans_A, trans_B)


def csrmv_op(node_A, node_B, trans=False):
    return _csr(node_A, node_B, trans, False, True)


def csrmm_op(node_A, node_B, trans_A=False, trans_B=False):
    return _csr(node_A, node_B, trans_A, trans_B, False)
