"""Which ops the CUDA backend executes; the partitioner's ``is_supported_fn``.

Superset of the reference table (cuda_compiler/op_support.py:9-60): every op
listed there is supported here, plus the extra ops ``op_classify`` knows.  The
callback signature ``(op_type, attrs)`` is the partitioner's
(npu_compiler/partitioner.py:42).
"""

from __future__ import annotations

from cuda_compiler.op_classify import _OP_CATEGORY_TABLE

_CUDA_SUPPORTED_OPS: set[str] = set(_OP_CATEGORY_TABLE)


def is_cuda_op_supported(op_type: str, _attrs: dict | None = None) -> bool:
    return op_type in _CUDA_SUPPORTED_OPS


def get_cuda_supported_ops() -> frozenset[str]:
    return frozenset(_CUDA_SUPPORTED_OPS)
