"""Partitioner / IR reader contract (reference: tests/test_partitioner.py)."""

from helpers import graph, node, ts
from npu_compiler import TransferOp, Partition, load_ir_from_dict, partition


def _ir():
    n = [node("a", "aten.relu.default", [ts("x", [4])], [ts("a", [4])]),
         node("b", "aten.weird.default", [ts("a", [4])], [ts("b", [4])]),
         node("c", "aten.relu.default", [ts("b", [4])], [ts("c", [4])]),
         node("d", "aten.add.Tensor", [ts("c", [4]), ts("a", [4])], [ts("d", [4])])]
    return graph(n, [ts("x", [4])], [ts("d", [4])])


def test_grouping_and_transfers():
    ir = _ir()
    plan = partition(ir, lambda op, attrs=None: op != "aten.weird.default")
    kinds = [(type(s).__name__, getattr(s, "target", getattr(s, "direction", None))) for s in plan.steps]
    assert kinds == [("Partition", "npu"), ("TransferOp", "to_cpu"), ("Partition", "cpu"), ("TransferOp", "to_npu"), ("Partition", "npu")]
    parts = [s for s in plan.steps if isinstance(s, Partition)]
    assert [p.partition_id for p in parts] == [0, 1, 2]
    assert parts[0].output_names == ["a"] and parts[1].input_names == ["a"] and parts[1].output_names == ["b"]
    assert parts[2].input_names == ["a", "b"] and parts[2].output_names == ["d"]
    transfers = [s for s in plan.steps if isinstance(s, TransferOp)]
    assert transfers[0].tensor_names == ["a"] and transfers[1].tensor_names == ["a", "b"]
    assert plan.original_ir is ir


def test_all_supported_single_partition():
    plan = partition(_ir(), lambda op, attrs=None: True)
    assert len(plan.steps) == 1 and plan.steps[0].target == "npu" and plan.steps[0].output_names == ["d"]


def test_empty_graph():
    assert partition({"nodes": []}, lambda *a: True).steps == []


def test_ir_reader_defaults():
    g = load_ir_from_dict(_ir())
    assert g.model_name == "test" and g.nodes[1].op_type == "aten.weird.default"
    assert g.graph_inputs[0].dtype == "float32" and g.get_node_by_name("c").inputs[0].name == "b"
    assert g.get_node_by_name("nope") is None
