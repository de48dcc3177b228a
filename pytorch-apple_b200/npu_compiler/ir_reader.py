"""IR JSON -> in-memory graph.

Mirrors the schema and the public names of the reference loader
(npu_compiler/ir_reader.py:9-94): ``TensorSpec``, ``OpNode``, ``IRGraph``,
``load_ir`` and ``load_ir_from_dict``.  The IR is the output contract of the
third-party ``torch_to_ir`` exporter: a topologically sorted list of ATen-level
nodes whose tensor operands are full tensor specs and whose non-tensor
arguments sit in ``attrs`` under their ATen schema names.
"""

from __future__ import annotations

import json
from dataclasses import dataclass, field
from typing import Any


@dataclass
class TensorSpec:
    name: str
    shape: list[int]
    dtype: str = "float32"
    alloc_shape: list[int] | None = None
    transform_steps: list[dict] | None = None
    producer_node: str | None = None
    producer_output_idx: int = 0

    @classmethod
    def from_dict(cls, d: dict[str, Any]) -> "TensorSpec":
        return cls(
            name=d["name"],
            shape=list(d["shape"]),
            dtype=d.get("dtype", "float32"),
            alloc_shape=d.get("alloc_shape"),
            transform_steps=d.get("transform_steps"),
            producer_node=d.get("producer_node"),
            producer_output_idx=d.get("producer_output_idx", 0),
        )


@dataclass
class OpNode:
    name: str
    op_type: str
    inputs: list[TensorSpec]
    outputs: list[TensorSpec]
    attrs: dict = field(default_factory=dict)

    @classmethod
    def from_dict(cls, d: dict[str, Any]) -> "OpNode":
        return cls(
            name=d["name"],
            op_type=d["op_type"],
            inputs=[TensorSpec.from_dict(t) for t in d.get("inputs", [])],
            outputs=[TensorSpec.from_dict(t) for t in d.get("outputs", [])],
            attrs=dict(d.get("attrs") or {}),
        )


@dataclass
class IRGraph:
    model_name: str
    graph_inputs: list[TensorSpec]
    graph_outputs: list[TensorSpec]
    weights: list[TensorSpec]
    weight_name_mapping: dict[str, str]
    nodes: list[OpNode]
    constants: dict = field(default_factory=dict)

    def get_node_by_name(self, name: str) -> OpNode | None:
        return next((n for n in self.nodes if n.name == name), None)


def load_ir_from_dict(data: dict) -> IRGraph:
    """Build an :class:`IRGraph` from an already-parsed IR dict."""
    return IRGraph(
        model_name=data.get("model_name", "unknown"),
        graph_inputs=[TensorSpec.from_dict(t) for t in data["graph_inputs"]],
        graph_outputs=[TensorSpec.from_dict(t) for t in data["graph_outputs"]],
        weights=[TensorSpec.from_dict(t) for t in data["weights"]],
        weight_name_mapping=dict(data.get("weight_name_mapping") or {}),
        nodes=[OpNode.from_dict(n) for n in data["nodes"]],
        constants=dict(data.get("constants") or {}),
    )


def load_ir(path: str) -> IRGraph:
    """Read an IR JSON file."""
    with open(path) as fh:
        return load_ir_from_dict(json.load(fh))
