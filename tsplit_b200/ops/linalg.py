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


def _heads_to_plain(shape):
    """[N, T, H, d] (head layout) -> [N, H, T, d]."""
    return (shape[0], shape[2], shape[1], shape[3])


class BatchMatMulOp(Op):
    """``C = op(A) op(B)`` over the leading (batch) dimensions.

    ``heads_A`` / ``heads_B`` / ``heads_out``: that operand is 4-D and stored ``[N, T, H, d]`` — a
    ``[N, T, H * d]`` projection output viewed per head — instead of ``[N, H, T, d]``; the batch is then
    ``(N, H)`` and the matrix of batch ``(n, h)`` is ``x[n, :, h, :]``.  The reference's Transformer example
    transposes heads in and out around every attention product (``examples/transformer.py:131-159``); here the
    GEMM reads and writes the projection layout in place (``tsb_gemm_tf32_heads``), so those copies do not exist."""
    name = "BatchMatMul"

    def __call__(self, a, b, trans_A=False, trans_B=False, heads_A=False, heads_B=False, heads_out=False):
        return Op.__call__(self, a, b, trans_A=trans_A, trans_B=trans_B, heads_A=bool(heads_A),
                           heads_B=bool(heads_B), heads_out=bool(heads_out))

    @staticmethod
    def _layouts(node):
        return (node.attrs.get("heads_A", False), node.attrs.get("heads_B", False),
                node.attrs.get("heads_out", False))

    def np_compute(self, node, iv):
        a, b = iv
        la, lb, lc = self._layouts(node)
        if la:
            a = np.transpose(a, (0, 2, 1, 3))
        if lb:
            b = np.transpose(b, (0, 2, 1, 3))
        if node.attrs["trans_A"]:
            a = np.swapaxes(a, -1, -2)
        if node.attrs["trans_B"]:
            b = np.swapaxes(b, -1, -2)
        c = np.matmul(a, b)
        return np.ascontiguousarray(np.transpose(c, (0, 2, 1, 3))) if lc else c

    def gpu_compute(self, node, iv, out, stream):
        a, b = iv
        ta, tb = node.attrs["trans_A"], node.attrs["trans_B"]
        la, lb, lc = self._layouts(node)
        sa_shape = _heads_to_plain(a.shape) if la else a.shape
        sb_shape = _heads_to_plain(b.shape) if lb else b.shape
        m, n, k = _mm_shape(sa_shape, sb_shape, ta, tb)
        batch = 1
        for d in sa_shape[:-2]:
            batch *= d
        assert a.is_contiguous() and b.is_contiguous() and out.is_contiguous()
        if not (la or lb or lc):
            G.gemm(a, b, out, ta, tb, stream, batch=batch, m=m, n=n, k=k,
                   sa=a.shape[-1] * a.shape[-2], sb=b.shape[-1] * b.shape[-2], sc=m * n,
                   lda=a.shape[-1], ldb=b.shape[-1], ldc=n)
            return
        heads = sa_shape[1]
        # head layout [N, T, H, d]: rows are H * d apart, heads d apart
        lda, sa = (heads * a.shape[3], a.shape[3]) if la else (a.shape[-1], a.shape[-1] * a.shape[-2])
        ldb, sb = (heads * b.shape[3], b.shape[3]) if lb else (b.shape[-1], b.shape[-1] * b.shape[-2])
        ldc, sc = (heads * n, n) if lc else (n, m * n)
        G.gemm(a, b, out, ta, tb, stream, batch=batch, m=m, n=n, k=k, sa=sa, sb=sb, sc=sc, lda=lda, ldb=ldb, ldc=ldc,
               heads=heads, head_mask=int(la) | int(lb) << 1 | int(lc) << 2)

    def gradient(self, node, g):
        a, b = node.inputs
        ta, tb = node.attrs["trans_A"], node.attrs["trans_B"]
        la, lb, lc = self._layouts(node)

        def mm(x, y, tx, ty, lx, ly, lo):
            return batch_matmul_op(x, y, tx, ty, heads_A=lx, heads_B=ly, heads_out=lo)
        if not ta and not tb:
            return [mm(g, b, False, True, lc, lb, la), mm(a, g, True, False, la, lc, lb)]
        if ta and not tb:
            return [mm(b, g, False, True, lb, lc, la), mm(a, g, False, False, la, lc, lb)]
        if not ta and tb:
            return [mm(g, b, False, False, lc, lb, la), mm(g, a, True, False, lc, la, lb)]
        return [mm(b, g, True, True, lb, lc, la), mm(g, a, True, True, lc, la, lb)]

    def _plain_shapes(self, node, s):
        la, lb, _ = self._layouts(node)
        return (_heads_to_plain(s[0]) if la else tuple(s[0])), (_heads_to_plain(s[1]) if lb else tuple(s[1]))

    def infer_shape(self, node, s):
        sa, sb = self._plain_shapes(node, s)
        assert tuple(sa[:-2]) == tuple(sb[:-2]), "batch dims differ"
        m, n, _ = _mm_shape(sa, sb, node.attrs["trans_A"], node.attrs["trans_B"])
        if self._layouts(node)[2]:
            assert len(sa) == 4, "head layout needs 4-D operands"
            return (sa[0], m, sa[1], n)
        return tuple(sa[:-2]) + (m, n)

    def flops(self, node, s, out):
        sa, sb = self._plain_shapes(node, s)
        m, n, k = _mm_shape(sa, sb, node.attrs["trans_A"], node.attrs["trans_B"])
        b = 1
        for d in sa[:-2]:
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


def batch_matmul_op(node_A, node_B, trans_A=False, trans_B=False, heads_A=False, heads_B=False, heads_out=False):
    return _bmm(node_A, node_B, trans_A, trans_B, heads_A, heads_B, heads_out)


def csrmv_op(node_A, node_B, trans=False):
    return _csr(node_A, node_B, trans, False, True)


def csrmm_op(node_A, node_B, trans_A=False, trans_B=False):
    return _csr(node_A, node_B, trans_A, trans_B, False)
