"""IR object model of the exporter package (``torch_ir.ir``).

The reference builds these objects itself when it hands a host partition to the ATen
executor (npu_runtime/cpu_fallback.py:21-129: ``TensorMeta(name, shape, dtype, producer_node,
producer_output_idx)``, ``OpNode(name, op_type, inputs, outputs, attrs)``, ``IR(nodes,
graph_inputs, graph_outputs, weights, weight_name_mapping, model_name)``) and reads
``.nodes / .weights / .graph_inputs / .graph_outputs`` and ``.save(path)`` from what
``extract_ir`` returns (examples/extract_qwen_ir.py:137-151, 233-275).  ``save`` writes the
IR JSON schema that ``npu_compiler.ir_reader`` loads.
"""

from __future__ import annotations

import json
from dataclasses import dataclass, field
from typing import Any


@dataclass
class TensorMeta:
    name: str
    shape: list[int]
    dtype: str = "float32"
    producer_node: str | None = None
    producer_output_idx: int = 0

    def to_dict(self) -> dict[str, Any]:
        d: dict[str, Any] = {"name": self.name, "shape": [int(s) for s in self.shape], "dtype": self.dtype}
        if self.producer_node is not None:
            d["producer_node"] = self.producer_node
            d["producer_output_idx"] = int(self.producer_output_idx)
        return d

    @classmethod
    def from_dict(cls, d: dict[str, Any]) -> "TensorMeta":
        return cls(d["name"], list(d["shape"]), d.get("dtype", "float32"), d.get("producer_node"), d.get("producer_output_idx", 0))


@dataclass
class OpNode:
    name: str
    op_type: str
    inputs: list[TensorMeta]
    outputs: list[TensorMeta]
    attrs: dict = field(default_factory=dict)

    def to_dict(self) -> dict[str, Any]:
        return {"name": self.name, "op_type": self.op_type, "inputs": [t.to_dict() for t in self.inputs],
                "outputs": [t.to_dict() for t in self.outputs], "attrs": dict(self.attrs)}

    @classmethod
    def from_dict(cls, d: dict[str, Any]) -> "OpNode":
        return cls(d["name"], d["op_type"], [TensorMeta.from_dict(t) for t in d.get("inputs", [])],
                   [TensorMeta.from_dict(t) for t in d.get("outputs", [])], dict(d.get("attrs") or {}))


@dataclass
class IR:
    nodes: list[OpNode]
    graph_inputs: list[TensorMeta]
    graph_outputs: list[TensorMeta]
    weights: list[TensorMeta]
    weight_name_mapping: dict[str, str] = field(default_factory=dict)
    model_name: str = "model"
    constants: dict = field(default_factory=dict)

    def to_dict(self) -> dict[str, Any]:
        d = {"model_name": self.model_name, "graph_inputs": [t.to_dict() for t in self.graph_inputs],
             "graph_outputs": [t.to_dict() for t in self.graph_outputs], "weights": [t.to_dict() for t in self.weights],
             "weight_name_mapping": dict(self.weight_name_mapping), "nodes": [n.to_dict() for n in self.nodes]}
        if self.constants:
            d["constants"] = self.constants
        return d

    @classmethod
    def from_dict(cls, d: dict[str, Any]) -> "IR":
        return cls([OpNode.from_dict(n) for n in d["nodes"]], [TensorMeta.from_dict(t) for t in d["graph_inputs"]],
                   [TensorMeta.from_dict(t) for t in d["graph_outputs"]], [TensorMeta.from_dict(t) for t in d.get("weights", [])],
                   dict(d.get("weight_name_mapping") or {}), d.get("model_name", "model"), dict(d.get("constants") or {}))

    def save(self, path: str) -> None:
        with open(path, "w") as f:
            json.dump(self.to_dict(), f)

    @classmethod
    def load(cls, path: str) -> "IR":
        with open(path) as f:
            return cls.from_dict(json.load(f))
