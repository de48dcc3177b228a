"""CPU oracle: run an IR dict node by node on ATen, on the host.

TEST INFRASTRUCTURE - not part of the product.  Only the test-suite, the smoke
check and the CPU-baseline leg of the benchmark may import this module.

What it restates.  The reference's CPU path is
npu_runtime/cpu_fallback.py:32-175: partition nodes are wrapped into a
``torch_ir.IR`` and handed to ``torch_ir.IRExecutor(ir, weights).execute(inputs)``,
which dispatches every node to the ATen operator its ``op_type`` names, with the
node's tensor inputs as positional tensor arguments and ``attrs`` as the
schema-named remaining arguments.  ``torch_ir`` is the third-party package
``pytorch-ir`` pinned at 0.2.2 by the reference (pyproject.toml:9); it is not
vendored with the reference and is not installed here, so its published
behaviour - "execute each node with torch.ops.aten" - is restated below.  The
arithmetic itself is PyTorch's own ATen CPU kernels, the same ones the
reference path ends in.

Pinned against: the four known-answer graphs and the bf16 round trip of the
reference's tests/test_cpu_fallback.py:14-173 (tests/test_oracle.py), and eager
``model(x)`` of the exported ResNet / Qwen2 modules, bit for bit
(tests/golden/make_golden.py writes the fixtures).

numpy <-> torch conversion follows cpu_fallback.py:178-194: bf16 travels as
``ml_dtypes.bfloat16`` (or raw uint16) arrays and is reinterpreted, never cast.
"""

from __future__ import annotations

import operator
import re
from typing import Any, Sequence

import numpy as np
import torch

_TORCH_DTYPES = {
    "float32": torch.float32, "float16": torch.float16, "bfloat16": torch.bfloat16,
    "int32": torch.int32, "int64": torch.int64, "bool": torch.bool, "float64": torch.float64,
    "uint8": torch.uint8, "int8": torch.int8, "int16": torch.int16,
}


def numpy_to_torch(arr: np.ndarray) -> torch.Tensor:
    """cpu_fallback.py:178-185."""
    arr = np.asarray(arr)
    if arr.dtype == np.uint16:
        return torch.from_numpy(arr.copy()).view(torch.bfloat16)
    if arr.dtype.name == "bfloat16":
        return torch.from_numpy(arr.view(np.uint16).copy()).view(torch.bfloat16)
    return torch.from_numpy(arr.copy())


def torch_to_numpy(t: torch.Tensor) -> np.ndarray:
    """cpu_fallback.py:187-194."""
    import ml_dtypes

    t = t.detach().cpu()
    if t.dtype == torch.bfloat16:
        return t.contiguous().view(torch.uint16).numpy().view(ml_dtypes.bfloat16).copy()
    return t.numpy().copy()


def _parse_attr(value: Any) -> Any:
    """Attribute values that were stringified for JSON (dtypes, devices, layouts)."""
    if isinstance(value, str):
        m = re.fullmatch(r"torch\.(\w+)", value)
        if m and hasattr(torch, m.group(1)):
            return getattr(torch, m.group(1))
        if value in ("cpu", "meta") or value.startswith("cuda"):
            return torch.device("cpu")
    return value


def _resolve_op(op_type: str):
    m = re.fullmatch(r"aten\.(\w+)\.(\w+)", op_type)
    if not m:
        return None
    packet = getattr(torch.ops.aten, m.group(1))
    return getattr(packet, m.group(2))


def _rope_tables(inv_freq: torch.Tensor, position_ids: torch.Tensor, out_dtype: torch.dtype):
    """Body of the ``wrap_with_set_grad_enabled`` node of the Qwen2 graphs: the
    rotary-embedding table.  fp32 outer product of ``inv_freq`` and positions,
    duplicated along the last axis, cos/sin, cast to the activation dtype
    (the correct statement of the op the reference's rope kernels compute,
    metal_kernels/rope.metal:34-44; the sub-graph itself was read from
    ``torch.export`` of the reference's wrappers)."""
    b = position_ids.shape[0]
    inv = inv_freq[None, :, None].float().expand(b, -1, 1)
    pos = position_ids[:, None, :].float()
    freqs = (inv @ pos).transpose(1, 2)
    emb = torch.cat((freqs, freqs), dim=-1)
    return (emb.cos() * 1.0).to(out_dtype), (emb.sin() * 1.0).to(out_dtype)


class IRInterpreter:
    """``IRInterpreter(ir_dict, weights).execute(inputs) -> dict name -> Tensor``.

    ``weights`` maps state-dict key *or* placeholder name to a tensor/ndarray.
    ``dtype_override`` (e.g. ``torch.float32``) runs a low-precision IR with every
    floating tensor widened - the "fp32 on the CPU path" arm of the ResNet configs
    is simply the fp32 IR, so this is only a diagnostic aid.
    """

    def __init__(self, ir: dict, weights: dict[str, Any]):
        self.ir = ir
        self.nodes = ir["nodes"]
        mapping = ir.get("weight_name_mapping") or {}
        key_to_ph = {}
        for ph, key in mapping.items():
            key_to_ph.setdefault(key, []).append(ph)
        self.env0: dict[str, torch.Tensor] = {}
        consts = ir.get("constants") or {}
        for spec in ir.get("weights", []):
            key = spec["name"]
            names = key_to_ph.get(key, []) + [key]
            val = None
            for n in names:
                if n in weights:
                    val = weights[n]
                    break
            if val is None and key in consts:
                c = consts[key]
                val = torch.tensor(c["data"], dtype=_TORCH_DTYPES[c["dtype"]]).reshape(c["shape"])
            if val is None:
                continue
            t = val if isinstance(val, torch.Tensor) else numpy_to_torch(val)
            for n in names:
                self.env0[n] = t
        # Intermediates are dropped after their last reader (a 28-layer decode step at batch 64 would
        # otherwise hold ~50 GB of repeated K/V); results are unaffected.
        keep = {o["name"] for o in ir["graph_outputs"]}
        last: dict[str, int] = {}
        for i, node in enumerate(self.nodes):
            for t in node.get("inputs", []):
                last[t["name"]] = i
        self._dead_after: dict[int, list[str]] = {}
        for name, i in last.items():
            if name not in keep and name not in self.env0:
                self._dead_after.setdefault(i, []).append(name)

    def execute(self, inputs: dict[str, Any] | Sequence[Any], keep_all: bool = False) -> dict[str, torch.Tensor]:
        env = dict(self.env0)
        if not isinstance(inputs, dict):
            inputs = {s["name"]: v for s, v in zip(self.ir["graph_inputs"], inputs)}
        for k, v in inputs.items():
            env[k] = v if isinstance(v, torch.Tensor) else numpy_to_torch(v)
        with torch.no_grad():
            for i, node in enumerate(self.nodes):
                self._run_node(node, env)
                if not keep_all:
                    for name in self._dead_after.get(i, ()):
                        env.pop(name, None)
        if keep_all:
            return env
        return {o["name"]: env[o["name"]] for o in self.ir["graph_outputs"]}

    # ------------------------------------------------------------------
    def _run_node(self, node: dict, env: dict) -> None:
        op = node["op_type"]
        ins = [env[t["name"]] for t in node.get("inputs", [])]
        outs = node.get("outputs", [])
        attrs = {k: _parse_attr(v) for k, v in (node.get("attrs") or {}).items()}
        if op == "aten._assert_tensor_metadata.default" or not outs:
            return
        if op == str(operator.getitem):
            env[outs[0]["name"]] = ins[attrs.get("index", 0)]
            return
        if op == "wrap_with_set_grad_enabled":
            cos, sin = _rope_tables(ins[0], ins[1], _TORCH_DTYPES[outs[0]["dtype"]])
            env[outs[0]["name"]], env[outs[1]["name"]] = cos, sin
            return
        if op == "aten.detach_.default":  # in-place detach is refused on views; the value is the same
            env[outs[0]["name"]] = ins[0].detach()
            return
        fn = _resolve_op(op)
        if fn is None:
            raise ValueError(f"oracle: unknown op_type {op!r}")
        result = self._call(fn, ins, attrs)
        if isinstance(result, (tuple, list)):
            for spec, r in zip(outs, result):
                env[spec["name"]] = r
        else:
            env[outs[0]["name"]] = result

    @staticmethod
    def _call(fn, tensors: list[torch.Tensor], attrs: dict):
        """Bind tensors positionally to the schema's tensor-typed parameters (list
        parameters swallow every remaining tensor), attrs by name."""
        args, kwargs = [], {}
        it = iter(tensors)
        left = len(tensors)
        for a in fn._schema.arguments:
            tname = str(a.type)
            if a.name in attrs:
                val = attrs[a.name]
            elif tname in ("Tensor", "Optional[Tensor]") and left > 0:
                val = next(it); left -= 1
            elif tname in ("List[Tensor]", "List[Optional[Tensor]]") and left > 0:
                val = list(it); left = 0
            else:
                continue
            if a.name == "device":
                continue
            if a.kwarg_only:
                kwargs[a.name] = val
            else:
                args.append((a.name, val))
        # positional arguments must be contiguous from the left; pass the rest by name
        pos, names = [], [a.name for a in fn._schema.arguments if not a.kwarg_only]
        for (name, val), expect in zip(args, names):
            if name != expect:
                break
            pos.append(val)
        for name, val in args[len(pos):]:
            kwargs[name] = val
        return fn(*pos, **kwargs)


def run_ir(ir: dict, weights: dict[str, Any], inputs) -> dict[str, np.ndarray]:
    """Convenience: execute and return numpy outputs (bf16 as ml_dtypes arrays)."""
    return {k: torch_to_numpy(v) for k, v in IRInterpreter(ir, weights).execute(inputs).items()}


def execute_cpu_partition(partition_nodes: list[dict], tensor_pool: dict[str, np.ndarray],
                          weights: dict[str, np.ndarray], weight_name_mapping: dict[str, str] | None = None):
    """Same signature and result as the reference's
    ``npu_runtime.cpu_fallback.execute_cpu_partition`` (cpu_fallback.py:32-69):
    returns every tensor the partition's nodes produce."""
    made = [t for n in partition_nodes for t in n.get("outputs", [])]
    made_names = {t["name"] for t in made}
    ext = {}
    for n in partition_nodes:
        for t in n.get("inputs", []):
            if t["name"] not in made_names:
                ext.setdefault(t["name"], t)
    wnames = set(weights) | set(weight_name_mapping or {})
    ir = {
        "model_name": "cpu_partition",
        "graph_inputs": [t for k, t in ext.items() if k not in wnames],
        "graph_outputs": made,
        "weights": [t for k, t in ext.items() if k in wnames],
        "weight_name_mapping": {},
        "nodes": partition_nodes,
    }
    w = {}
    for t in ir["weights"]:
        k = t["name"]
        if k in weights:
            w[k] = weights[k]
        elif weight_name_mapping and weight_name_mapping.get(k) in weights:
            w[k] = weights[weight_name_mapping[k]]
    out = IRInterpreter(ir, w).execute({t["name"]: tensor_pool[t["name"]] for t in ir["graph_inputs"]})
    return {k: torch_to_numpy(v) for k, v in out.items()}


def cpu_executor_factory(nodes, weights, mapping):
    """Adapter for ``DAGExecutor(cpu_executor_factory=...)`` in tests."""
    return lambda pool: execute_cpu_partition(nodes, pool, weights, mapping)
