"""Shared builders for the tests: tiny IR graphs and seeded model cases."""

from __future__ import annotations

import numpy as np
import torch


def ts(name, shape, dtype="float32"):
    return {"name": name, "shape": list(shape), "dtype": dtype}


def node(name, op, inputs, outputs, **attrs):
    outs = [dict(o, producer_node=name, producer_output_idx=i) for i, o in enumerate(outputs)]
    return {"name": name, "op_type": op, "inputs": list(inputs), "outputs": outs, "attrs": attrs}


def graph(nodes, inputs, outputs, weights=(), mapping=None, name="test"):
    return {"model_name": name, "graph_inputs": list(inputs), "graph_outputs": list(outputs), "weights": list(weights),
            "weight_name_mapping": dict(mapping or {}), "nodes": list(nodes)}


def to_f32(x) -> np.ndarray:
    if isinstance(x, torch.Tensor):
        return x.detach().float().cpu().numpy()
    if hasattr(x, "to_numpy"):
        x = x.to_numpy()
    return np.asarray(x).astype(np.float32)


def rmsnorm_graph(rows, cols, dtype="bfloat16", eps=1e-6):
    """The 8-node chain the Qwen2 exporter emits for one RMSNorm."""
    f32 = "float32"
    x, w = ts("x", [rows, cols], dtype), ts("w", [cols], dtype)
    n = [
        node("to_a", "aten.to.dtype", [x], [ts("to_a", [rows, cols], f32)], dtype="torch.float32"),
        node("pow_1", "aten.pow.Tensor_Scalar", [ts("to_a", [rows, cols], f32)], [ts("pow_1", [rows, cols], f32)], exponent=2),
        node("mean", "aten.mean.dim", [ts("pow_1", [rows, cols], f32)], [ts("mean", [rows, 1], f32)], dim=[-1], keepdim=True),
        node("add", "aten.add.Tensor", [ts("mean", [rows, 1], f32)], [ts("add", [rows, 1], f32)], other=eps),
        node("rsqrt", "aten.rsqrt.default", [ts("add", [rows, 1], f32)], [ts("rsqrt", [rows, 1], f32)]),
        node("mul_a", "aten.mul.Tensor", [ts("to_a", [rows, cols], f32), ts("rsqrt", [rows, 1], f32)], [ts("mul_a", [rows, cols], f32)]),
        node("to_b", "aten.to.dtype", [ts("mul_a", [rows, cols], f32)], [ts("to_b", [rows, cols], dtype)], dtype="torch." + dtype),
        node("y", "aten.mul.Tensor", [w, ts("to_b", [rows, cols], dtype)], [ts("y", [rows, cols], dtype)]),
    ]
    return graph(n, [x], [ts("y", [rows, cols], dtype)], [w])


def silu_mul_graph(rows, cols, dtype="bfloat16"):
    g, u = ts("gate", [rows, cols], dtype), ts("up", [rows, cols], dtype)
    n = [node("silu", "aten.silu.default", [g], [ts("silu", [rows, cols], dtype)]),
         node("y", "aten.mul.Tensor", [ts("silu", [rows, cols], dtype), u], [ts("y", [rows, cols], dtype)])]
    return graph(n, [g, u], [ts("y", [rows, cols], dtype)])


def masked_softmax_graph(heads, T, dtype="bfloat16"):
    """scores [1,H,T,T] + mask [1,1,T,T] -> softmax(fp32) -> cast, as in the attention block."""
    s, m = ts("scores", [1, heads, T, T], dtype), ts("mask", [1, 1, T, T], dtype)
    n = [node("add", "aten.add.Tensor", [s, m], [ts("add", [1, heads, T, T], dtype)]),
         node("softmax", "aten.softmax.int", [ts("add", [1, heads, T, T], dtype)], [ts("softmax", [1, heads, T, T], "float32")],
              dim=-1, dtype="torch.float32"),
         node("y", "aten.to.dtype", [ts("softmax", [1, heads, T, T], "float32")], [ts("y", [1, heads, T, T], dtype)],
              dtype="torch." + dtype)]
    return graph(n, [s, m], [ts("y", [1, heads, T, T], dtype)])


def rope_graph(H, T, D=128, dtype="bfloat16"):
    """RoPE table (HOP node) + rotate chain on x [1,H,T,D], as the Qwen2 exporter emits them."""
    x = ts("x", [1, H, T, D], dtype)
    inv, pos = ts("inv_freq", [D // 2], "float32"), ts("position_ids", [1, T], "int64")
    cs = lambda n: ts(n, [1, T, D], dtype)
    u = lambda n: ts(n, [1, 1, T, D], dtype)
    h = lambda n: ts(n, [1, H, T, D // 2], dtype)
    f = lambda n: ts(n, [1, H, T, D], dtype)
    n = [
        node("hop", "wrap_with_set_grad_enabled", [inv, pos], [cs("hop_0"), cs("hop_1")]),
        node("cos", "<built-in function getitem>", [cs("hop_0"), cs("hop_1")], [cs("cos")], index=0),
        node("sin", "<built-in function getitem>", [cs("hop_0"), cs("hop_1")], [cs("sin")], index=1),
        node("cos_u", "aten.unsqueeze.default", [cs("cos")], [u("cos_u")], dim=1),
        node("sin_u", "aten.unsqueeze.default", [cs("sin")], [u("sin_u")], dim=1),
        node("mul_c", "aten.mul.Tensor", [x, u("cos_u")], [f("mul_c")]),
        node("lo", "aten.slice.Tensor", [x], [h("lo")], dim=3, start=0, end=D // 2),
        node("hi", "aten.slice.Tensor", [x], [h("hi")], dim=3, start=D // 2, end=9223372036854775807),
        node("neg", "aten.neg.default", [h("hi")], [h("neg")]),
        node("cat", "aten.cat.default", [h("neg"), h("lo")], [f("cat")], dim=-1),
        node("mul_s", "aten.mul.Tensor", [f("cat"), u("sin_u")], [f("mul_s")]),
        node("y", "aten.add.Tensor", [f("mul_c"), f("mul_s")], [f("y")]),
    ]
    return graph(n, [x, pos], [f("y")], [inv])


def run_backend(ir, weights, inputs, compile_kwargs=None):
    """IR -> partition -> DAGExecutor on the CUDA backend -> dict of float32 numpy outputs (plus raw)."""
    from functools import partial

    from cuda_compiler import compile_subgraph, is_cuda_op_supported
    from cuda_runtime import CUDABackend
    from npu_compiler import partition
    from npu_runtime import DAGExecutor

    plan = partition(ir, is_cuda_op_supported)
    dag = DAGExecutor(plan, CUDABackend(), partial(compile_subgraph, **(compile_kwargs or {})))
    dag.load_weights(weights)
    out = dag.execute(inputs)
    return {k: (v if isinstance(v, np.ndarray) else v.to_numpy()) for k, v in out.items()}, dag


def np_inputs(ir, tensors):
    from oracle.ir_interpreter import torch_to_numpy

    return {s["name"]: torch_to_numpy(t) for s, t in zip(ir["graph_inputs"], tensors)}
