"""ATen op -> lowering category.

Same categories and the same assignment for every op the reference classifies
(cuda_compiler/op_classify.py:17-79); unknown ops fall into SPECIAL as there.
A few ops that newer exporters emit around the same graphs are added
(``lift_fresh_copy``, ``sub``, ``sigmoid``, ``argmax``, ...).
"""

from __future__ import annotations

from enum import Enum, auto


class OpCategory(Enum):
    ANCHOR_BLAS = auto()  # dense contraction: fusion barrier, tensor-core kernel
    ELEMENTWISE = auto()  # can be chained into one elementwise kernel
    REDUCTION = auto()    # row reduction / pooling / normalisation kernel
    SHAPE_ALIAS = auto()  # view of an existing buffer, no launch when expressible as strides
    SPECIAL = auto()      # gather/scatter/rope/fill
    NOOP = auto()         # metadata asserts


_BLAS = ("aten.matmul.default", "aten.linear.default", "aten.addmm.default", "aten.conv2d.default",
         "aten.mm.default", "aten.bmm.default")
_ELEMENTWISE = (
    "aten.relu.default", "aten.relu_.default", "aten.silu.default", "aten.add.Tensor", "aten.add_.Tensor",
    "aten.mul.Tensor", "aten.div.Tensor", "aten.neg.default", "aten.pow.Tensor_Scalar", "aten.rsqrt.default",
    "aten.cos.default", "aten.sin.default",
    "aten.sub.Tensor", "aten.sigmoid.default", "aten.exp.default", "aten.sqrt.default", "aten.tanh.default",
    "aten.gelu.default", "aten.silu_.default", "aten.mul_.Tensor",
)
_REDUCTION = ("aten.softmax.int", "aten.mean.dim", "aten.batch_norm.default", "aten.max_pool2d.default",
              "aten.adaptive_avg_pool2d.default", "aten._softmax.default", "aten.argmax.default")
_ALIAS = (
    "aten.reshape.default", "aten.view.default", "aten.flatten.using_ints", "aten.contiguous.default",
    "aten.unsqueeze.default", "aten.alias.default", "aten.detach_.default", "aten.to.dtype", "aten.dropout.default",
    "<built-in function getitem>", "aten.t.default", "aten.expand.default", "aten.slice.Tensor", "aten.transpose.int",
    "aten.cat.default",
    "aten.lift_fresh_copy.default", "aten.detach.default", "aten.squeeze.dim", "aten.permute.default",
    "aten._to_copy.default", "aten.clone.default", "aten._unsafe_view.default",
)
_SPECIAL = ("aten.embedding.default", "wrap_with_set_grad_enabled", "aten.index_copy.default", "aten.full.default")
_NOOP = ("aten._assert_tensor_metadata.default",)

_OP_CATEGORY_TABLE: dict[str, OpCategory] = {}
for _ops, _cat in ((_BLAS, OpCategory.ANCHOR_BLAS), (_ELEMENTWISE, OpCategory.ELEMENTWISE),
                   (_REDUCTION, OpCategory.REDUCTION), (_ALIAS, OpCategory.SHAPE_ALIAS),
                   (_SPECIAL, OpCategory.SPECIAL), (_NOOP, OpCategory.NOOP)):
    for _op in _ops:
        _OP_CATEGORY_TABLE[_op] = _cat


def classify_op(op_type: str) -> OpCategory:
    return _OP_CATEGORY_TABLE.get(op_type, OpCategory.SPECIAL)
