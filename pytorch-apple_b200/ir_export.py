"""``nn.Module`` -> IR dict in the ``torch_to_ir`` JSON schema.

The reference obtains its IR from the third-party exporter
``torch_ir.extract_ir(model, example_inputs, model_name)`` (used at
examples/extract_qwen_ir.py:29 and tests/test_dag_executor.py:51-70).  This
module produces the same schema with ``torch.export`` so that models can be
lowered without that package:

* one node per FX ``call_function`` in topological order, ``op_type`` being the
  string form of the target (``aten.linear.default``,
  ``<built-in function getitem>``, ``wrap_with_set_grad_enabled``);
* tensor arguments, in call order and with list arguments flattened, become
  ``inputs``; every other argument goes to ``attrs`` under its ATen schema name;
* parameters and buffers become ``weights`` named by state-dict key, with
  ``weight_name_mapping`` from FX placeholder to that key;
* a ``getitem`` node lists all outputs of the producing node as inputs and
  selects with ``attrs["index"]``, which is what the reference analyzer expects
  (cuda_compiler/subgraph_analyzer.py:586-595).

Small tensors that export lifts into constants are emitted as weights whose
values are stored inline under ``constants``.
"""

from __future__ import annotations

import json
import operator
from typing import Any, Sequence

import torch

_DTYPE_NAMES = {
    torch.float32: "float32", torch.float16: "float16", torch.bfloat16: "bfloat16",
    torch.int32: "int32", torch.int64: "int64", torch.bool: "bool", torch.float64: "float64",
    torch.uint8: "uint8", torch.int8: "int8", torch.int16: "int16",
}


def _spec(name: str, val: torch.Tensor, producer: str | None = None, idx: int = 0) -> dict:
    d = {"name": name, "shape": [int(s) for s in val.shape], "dtype": _DTYPE_NAMES.get(val.dtype, str(val.dtype))}
    if producer is not None:
        d["producer_node"] = producer
        d["producer_output_idx"] = idx
    return d


def _jsonable(v: Any) -> Any:
    if isinstance(v, (list, tuple)):
        return [_jsonable(x) for x in v]
    if isinstance(v, (torch.SymInt,)):
        return int(v)
    try:
        json.dumps(v)
        return v
    except (TypeError, ValueError):
        return str(v)


def _output_specs(node: torch.fx.Node) -> list[dict]:
    val = node.meta.get("val")
    if isinstance(val, torch.Tensor):
        return [_spec(node.name, val, node.name, 0)]
    if isinstance(val, (tuple, list)):
        return [_spec(f"{node.name}_{i}", v, node.name, i) for i, v in enumerate(val) if isinstance(v, torch.Tensor)]
    return []


def extract_ir(model: torch.nn.Module, example_inputs: Sequence[torch.Tensor], model_name: str = "model") -> dict:
    """Export ``model`` (meta-device models are fine) and return the IR dict."""
    ep = torch.export.export(model, tuple(example_inputs), strict=False)
    sig = ep.graph_signature
    kinds = {s.arg.name: s for s in sig.input_specs if hasattr(s.arg, "name")}

    tensors: dict[str, list[dict]] = {}  # fx node name -> its output specs
    graph_inputs, weights, mapping, constants = [], [], {}, {}
    nodes: list[dict] = []

    for node in ep.graph.nodes:
        if node.op == "placeholder":
            val = node.meta.get("val")
            if not isinstance(val, torch.Tensor):
                continue
            spec = kinds.get(node.name)
            kind = spec.kind.name if spec is not None else "USER_INPUT"
            tensors[node.name] = [_spec(node.name, val)]
            if kind == "USER_INPUT":
                graph_inputs.append(_spec(node.name, val))
            else:
                key = spec.target or node.name
                weights.append(_spec(key, val))
                mapping[node.name] = key
                if kind == "CONSTANT_TENSOR":
                    const = ep.constants.get(key)
                    if isinstance(const, torch.Tensor) and const.device.type != "meta" and const.numel() <= 4096:
                        constants[key] = {"shape": list(const.shape), "dtype": _DTYPE_NAMES.get(const.dtype, str(const.dtype)),
                                          "data": const.detach().cpu().flatten().tolist()}
                    elif isinstance(val, torch.Tensor) and val.numel() == 0:
                        constants[key] = {"shape": list(val.shape), "dtype": _DTYPE_NAMES.get(val.dtype, str(val.dtype)), "data": []}
        elif node.op == "call_function":
            outs = _output_specs(node)
            tensors[node.name] = outs
            inputs: list[dict] = []
            attrs: dict[str, Any] = {}

            def take(arg, name):
                if isinstance(arg, torch.fx.Node):
                    src = tensors.get(arg.name)
                    if src:
                        inputs.extend(src if node.target is operator.getitem else src[:1])
                    return
                if isinstance(arg, (list, tuple)) and any(isinstance(a, torch.fx.Node) for a in arg):
                    for a in arg:
                        take(a, name)
                    return
                if name is not None:
                    attrs[name] = _jsonable(arg)

            schema = getattr(node.target, "_schema", None)
            if node.target is operator.getitem:
                take(node.args[0], None)
                attrs["index"] = int(node.args[1])
            elif schema is not None:
                names = [a.name for a in schema.arguments]
                for i, arg in enumerate(node.args):
                    take(arg, names[i] if i < len(names) else f"arg{i}")
                for k, arg in node.kwargs.items():
                    take(arg, k)
            else:  # higher-order op: keep tensor operands only
                for arg in node.args:
                    if isinstance(arg, torch.fx.Node) and arg.op != "get_attr":
                        take(arg, None)
            nodes.append({"name": node.name, "op_type": str(node.target), "inputs": inputs, "outputs": outs, "attrs": attrs})
        elif node.op == "output":
            flat = node.args[0] if isinstance(node.args[0], (list, tuple)) else [node.args[0]]
            graph_outputs = []
            for a in flat:
                if isinstance(a, torch.fx.Node) and tensors.get(a.name):
                    graph_outputs.append(dict(tensors[a.name][0]))

    return {
        "model_name": model_name,
        "graph_inputs": graph_inputs,
        "graph_outputs": graph_outputs,
        "weights": weights,
        "weight_name_mapping": mapping,
        "nodes": nodes,
        "constants": constants,
    }


def save_ir(ir: dict, path: str) -> None:
    with open(path, "w") as fh:
        json.dump(ir, fh)
