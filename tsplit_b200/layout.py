"""Physical-layout resolution for 4-D tensors on a CUDA context.

Logical shapes are always NCHW.  A 4-D array is stored channels-last when it
flows through image operators (the tensor-core convolution, pooling and
batch-norm kernels read channel-contiguous pixels) and row-major otherwise
(e.g. the [batch, heads, T, d] tensors of attention, which feed the batched
GEMM).  Element-wise and data-movement operators follow their input.
"""
from __future__ import annotations

IMAGE_OPS = {
    "Conv2d", "Conv2dGradData", "Conv2dGradFilter", "Conv2dBroadcastTo", "MaxPool2d", "AvgPool2d",
    "MaxPool2dGradient", "AvgPool2dGradient", "BatchNorm", "BatchNormGradient", "BatchNormGradData",
    "BatchNormGradScale", "BatchNormGradBias", "BatchNormRelu", "BatchNormReluGradient",
}
FOLLOW_OPS = {
    "Add", "AddBroadcast", "Mul", "Div", "ReluGradient", "AddRelu", "ReluOutGradient", "AddConst", "MulConst", "DivConst", "Opposite", "Sqrt", "Rsqrt",
    "Sigmoid", "Tanh", "Relu", "Where", "OnesLike", "ZerosLike", "Dropout", "DropoutGradient", "Concat",
    "ConcatGradient", "Slice", "SliceGradient", "Pad", "PadGradient", "Split", "SwapIn", "SwapOut",
}
LIKE_OPS = {"ReshapeGradient", "AvgPool2dGradient", "EmbeddingLookUpGradient"}


def resolve(topo_order, shapes):
    """node -> True when its value should be stored channels-last."""
    users = {}
    for n in topo_order:
        for i in n.inputs:
            users.setdefault(i, []).append(n)
    out = {}
    for n in topo_order:
        shp = shapes.get(n)
        if shp is None or len(shp) != 4:
            out[n] = False
            continue
        name = n.op.name
        if name == "Placeholder":
            out[n] = any(u.op.name in IMAGE_OPS for u in users.get(n, []))
        elif name in IMAGE_OPS:
            out[n] = True
        elif name in LIKE_OPS and n.attrs.get("like") is not None:
            out[n] = out.get(n.attrs["like"], False)
        elif name in FOLLOW_OPS:
            out[n] = any(out.get(i, False) for i in n.inputs
                         if shapes.get(i) is not None and len(shapes[i]) == 4)
        else:
            out[n] = False
    return out
