"""Stand-in for the third-party exporter package ``pytorch-ir`` (imported as ``torch_ir``).

The reference pins that package (pyproject.toml:9) and imports it at module level
(npu_runtime/cpu_fallback.py:17-18, tests/test_dag_executor.py:17), so without it neither
its orchestrator nor its tests import.  This package offers the surface they touch -
``IR``, ``IRExecutor``, ``extract_ir`` and ``torch_ir.ir.{OpNode, TensorMeta}`` - on top of
``torch.export``, so that the reference's ``DAGExecutor`` runs unmodified with this
repository's CUDA backend.  Put this directory's parent on ``sys.path`` to use it.
"""

from __future__ import annotations

from typing import Any, Sequence

from torch_ir.executor import IRExecutor
from torch_ir.ir import IR, OpNode, TensorMeta


def extract_ir(model, example_inputs: Sequence[Any], model_name: str = "model") -> IR:
    """Export ``model`` (meta-device modules and inputs are fine) and return its IR object."""
    from ir_export import extract_ir as _extract_dict

    return IR.from_dict(_extract_dict(model, tuple(example_inputs), model_name))


__all__ = ["IR", "IRExecutor", "OpNode", "TensorMeta", "extract_ir"]
