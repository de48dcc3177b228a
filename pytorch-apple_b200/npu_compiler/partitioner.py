"""Split an IR node list into device ("npu") and host ("cpu") partitions.

Interface and results follow the reference partitioner
(npu_compiler/partitioner.py:15-143): nodes arrive topologically sorted, each
is tagged by ``is_supported_fn(op_type, attrs)``, runs of equal tags become
``Partition`` objects with sequential ids, and a ``TransferOp`` is placed in
front of a partition whose predecessor ran on the other side, listing (sorted)
the tensors it needs from any earlier partition.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from itertools import groupby
from typing import Callable, Literal


@dataclass
class Partition:
    partition_id: int
    target: Literal["npu", "cpu"]
    nodes: list[dict]
    input_names: list[str] = field(default_factory=list)
    output_names: list[str] = field(default_factory=list)


@dataclass
class TransferOp:
    tensor_names: list[str]
    direction: Literal["to_cpu", "to_npu"]


@dataclass
class PartitionPlan:
    steps: list[Partition | TransferOp]
    original_ir: dict


def _names(node: dict, key: str) -> list[str]:
    return [t["name"] for t in node.get(key, [])]


def partition(ir_dict: dict, is_supported_fn: Callable[[str, dict | None], bool]) -> PartitionPlan:
    nodes = ir_dict.get("nodes", [])
    if not nodes:
        return PartitionPlan(steps=[], original_ir=ir_dict)

    def side(node: dict) -> str:
        return "npu" if is_supported_fn(node["op_type"], node.get("attrs")) else "cpu"

    parts: list[Partition] = []
    for target, run in groupby(nodes, key=side):
        parts.append(Partition(partition_id=len(parts), target=target, nodes=list(run)))

    # What every partition defines, and which partition defines each tensor.
    defined = [set(n for node in p.nodes for n in _names(node, "outputs")) for p in parts]
    owner = {name: i for i, names in enumerate(defined) for name in names}
    final_outputs = {t["name"] for t in ir_dict.get("graph_outputs", [])}

    exported: list[set[str]] = [set() for _ in parts]
    for i, p in enumerate(parts):
        needs = {n for node in p.nodes for n in _names(node, "inputs")} - defined[i]
        p.input_names = sorted(needs)
        for name in needs:
            src = owner.get(name)
            if src is not None and src != i:
                exported[src].add(name)
    for i, p in enumerate(parts):
        p.output_names = sorted(exported[i] | (defined[i] & final_outputs))

    steps: list[Partition | TransferOp] = []
    seen: set[str] = set()
    for i, p in enumerate(parts):
        if i > 0 and parts[i - 1].target != p.target:
            crossing = sorted(n for n in p.input_names if n in seen)
            if crossing:
                steps.append(TransferOp(crossing, "to_cpu" if p.target == "cpu" else "to_npu"))
        steps.append(p)
        seen |= defined[i]
    return PartitionPlan(steps=steps, original_ir=ir_dict)
