"""IR data model and graph partitioner shared by the compilers.

Only the two modules the CUDA path depends on live here: ``ir_reader`` (the
IR JSON schema as dataclasses) and ``partitioner`` (device/CPU segmentation).
"""

from npu_compiler.ir_reader import IRGraph, OpNode, TensorSpec, load_ir, load_ir_from_dict  # noqa: F401
from npu_compiler.partitioner import Partition, PartitionPlan, TransferOp, partition  # noqa: F401


def compute_strides(shape):
    """Row-major (C-contiguous) element strides of ``shape``.

    Same contract as the reference helper npu_compiler/codegen_ops.py:20-25,
    which is the only Metal-compiler symbol the CUDA path imports.
    """
    strides, acc = [], 1
    for extent in reversed(list(shape)):
        strides.append(acc)
        acc *= int(extent)
    return strides[::-1]
