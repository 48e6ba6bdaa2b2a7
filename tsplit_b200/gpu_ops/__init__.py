"""The user-facing ``ad`` namespace: ``from tsplit_b200 import gpu_ops as ad``.

Every name exported by the reference's ``python/athena/gpu_ops/__init__.py:1-116``
is here with the same signature, plus the executors the reference references but
does not ship (``microopExecutor``, ``capuchinExecutor``)."""
from ..graph import Node, Op, gradients, find_topo_sort, find_topo_sort2, sum_node_list, broadcast_rule
from ..ops.elementwise import (add_op, addbyconst_op, mul_op, mul_byconst_op, div_op, div_const_op,
                               opposite_op, sqrt_op, rsqrt_op, sigmoid_op, tanh_op, relu_op,
                               relu_gradient_op, where_op, add_relu_op, relu_out_gradient_op)
from ..ops.linalg import matmul_op, batch_matmul_op, csrmv_op, csrmm_op
from ..ops.conv import (conv2d_op, conv2d_gradient_of_data_op, conv2d_gradient_of_filter_op,
                        conv2d_broadcastto_op, conv2d_reducesum_op)
from ..ops.pool import max_pool2d_op, max_pool2d_gradient_op, avg_pool2d_op, avg_pool2d_gradient_op
from ..ops.norm import (batch_normalization_op, batch_normalization_gradient_op,
                        batch_normalization_gradient_of_data_op, batch_normalization_gradient_of_scale_op,
                        batch_normalization_gradient_of_bias_op, layer_normalization_op,
                        batch_normalization_relu_op)
from ..ops.shape import (array_reshape_op, array_reshape_gradient_op, transpose_op, slice_op,
                         slice_gradient_op, concat_op, concat_gradient_op, pad_op, pad_gradient_op,
                         broadcastto_op, broadcast_shape_op, broadcasttoTF_op, add_broadcast_op, reduce_sum_op,
                         reducesumaxiszero_op)
from ..ops.loss import (softmax_func, softmax_op, softmax_gradient_op, softmaxcrossentropy_op,
                        softmaxcrossentropy_gradient_op, masked_softmax_op, masked_softmax_gradient_op)
from ..ops.misc import (Variable, placeholder_op, oneslike_op, zeroslike_op, one_hot_op,
                        embedding_lookup_op, embedding_lookup_gradient_op, dropout_op, dropout_gradient_op,
                        swap_out_op, swap_in_op, split_op)
from ..executors import *          # noqa: F401,F403
from ..parallel.graph_hooks import (distributed_gradients, ps_gradients, distributed_communicate_op,   # noqa: E402
                                    ps_communicate_op)
