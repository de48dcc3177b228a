"""``IRExecutor``: runs an IR on the host with the ATen operator each node names.

This is the runner of *host partitions* - ops a caller's ``is_supported_fn`` keeps off the
GPU (docs/partitioning.md:33-40 of the reference) - with the calling convention the
reference's CPU fallback uses (npu_runtime/cpu_fallback.py:63-66, 154, 173-175):
``IRExecutor(ir, weights={name: Tensor}).execute((inputs...))`` returns the graph outputs
in ``ir.graph_outputs`` order.  Weights are looked up by the node-side name and, through
``ir.weight_name_mapping``, by state-dict key.
"""

from __future__ import annotations

import operator
import re
from typing import Any, Sequence

import torch

_ATEN = re.compile(r"aten\.(\w+)\.(\w+)")
_TORCH_NAME = re.compile(r"torch\.(\w+)")


def _attr_value(v: Any) -> Any:
    """Attributes survive a JSON round trip as strings: ``"torch.float32"`` -> dtype, device strings -> CPU."""
    if isinstance(v, str):
        m = _TORCH_NAME.fullmatch(v)
        if m and isinstance(getattr(torch, m.group(1), None), (torch.dtype, torch.layout, torch.memory_format)):
            return getattr(torch, m.group(1))
        if v in ("cpu", "meta") or v.startswith("cuda"):
            return torch.device("cpu")
    return v


def _rotary_tables(inv_freq: torch.Tensor, position_ids: torch.Tensor, dtype: torch.dtype):
    """The ``wrap_with_set_grad_enabled`` node of Qwen2-family exports: cos/sin tables of the rotary
    embedding - fp32 outer product of inverse frequencies and positions, both halves alike."""
    inv = inv_freq[None, :, None].float().expand(position_ids.shape[0], -1, 1)
    ang = (inv @ position_ids[:, None, :].float()).transpose(1, 2)
    ang = torch.cat((ang, ang), dim=-1)
    return ang.cos().to(dtype), ang.sin().to(dtype)


class IRExecutor:
    def __init__(self, ir, weights: dict[str, torch.Tensor] | None = None):
        self.ir = ir
        weights = dict(weights or {})
        mapping = getattr(ir, "weight_name_mapping", None) or {}
        self._consts: dict[str, torch.Tensor] = {}
        for w in ir.weights:
            t = weights.get(w.name)
            if t is None and w.name in mapping:
                t = weights.get(mapping[w.name])
            if t is None:
                for placeholder, key in mapping.items():
                    if key == w.name and placeholder in weights:
                        t = weights[placeholder]
                        break
            if t is not None:
                self._consts[w.name] = t
        for placeholder, key in mapping.items():      # nodes refer to weights by placeholder
            if placeholder not in self._consts:
                t = weights.get(placeholder, weights.get(key, self._consts.get(key)))
                if t is not None:
                    self._consts[placeholder] = t

    def execute(self, inputs: Sequence[torch.Tensor]) -> list[torch.Tensor]:
        values = dict(self._consts)
        if len(inputs) != len(self.ir.graph_inputs):
            raise ValueError(f"expected {len(self.ir.graph_inputs)} inputs, got {len(inputs)}")
        for meta, t in zip(self.ir.graph_inputs, inputs):
            values[meta.name] = t
        with torch.no_grad():
            for node in self.ir.nodes:
                self._run(node, values)
        return [values[o.name] for o in self.ir.graph_outputs]

    def _run(self, node, values: dict[str, torch.Tensor]) -> None:
        if not node.outputs or node.op_type == "aten._assert_tensor_metadata.default":
            return
        try:
            args = [values[t.name] for t in node.inputs]
        except KeyError as exc:
            raise RuntimeError(f"node '{node.name}': operand {exc} has no value") from None
        attrs = {k: _attr_value(v) for k, v in (node.attrs or {}).items()}
        if node.op_type == str(operator.getitem):
            values[node.outputs[0].name] = args[int(attrs.get("index", 0))]
            return
        if node.op_type == "wrap_with_set_grad_enabled":
            cos, sin = _rotary_tables(args[0], args[1], getattr(torch, node.outputs[0].dtype))
            values[node.outputs[0].name], values[node.outputs[1].name] = cos, sin
            return
        if node.op_type == "aten.detach_.default":
            values[node.outputs[0].name] = args[0].detach()
            return
        m = _ATEN.fullmatch(node.op_type)
        if m is None:
            raise ValueError(f"IRExecutor cannot run op_type {node.op_type!r}")
        op = getattr(getattr(torch.ops.aten, m.group(1)), m.group(2))
        result = op(**self._bind(op, args, attrs))
        if isinstance(result, (tuple, list)):
            for meta, r in zip(node.outputs, result):
                values[meta.name] = r
        else:
            values[node.outputs[0].name] = result

    @staticmethod
    def _bind(op, tensors: list[torch.Tensor], attrs: dict) -> dict[str, Any]:
        """Keyword arguments for ``op``: tensors fill the schema's tensor parameters in order (a
        tensor-list parameter takes all that remain), everything else comes from ``attrs`` by name."""
        kwargs: dict[str, Any] = {}
        rest = list(tensors)
        for arg in op._schema.arguments:
            kind = str(arg.type)
            if arg.name in attrs:
                if arg.name != "device":
                    kwargs[arg.name] = attrs[arg.name]
            elif kind in ("Tensor", "Optional[Tensor]") and rest:
                kwargs[arg.name] = rest.pop(0)
            elif kind in ("List[Tensor]", "List[Optional[Tensor]]") and rest:
                kwargs[arg.name], rest = rest, []
        return kwargs
