"""The executor-level cases of the reference's CUDA tests, through the same calls a caller of
the reference makes: ``compile_subgraph(ir_dict)`` -> ``CUDAExecutor(program)`` ->
``run({name: CUDABuffer}, weights)`` -> ``to_numpy()``; numpy references and tolerances as in
tests/test_cuda_executor.py:73-319 (buffers, backend, relu, silu*mul, GEMM, reshape, softmax) and
tests/test_cuda_fusion.py:81-374 (relu, neg, relu+add, silu*mul, add+relu, linear->relu, a tiny
gated MLP; rtol / atol 1e-1, seed 42).  The reference builds some programs from NVRTC source
strings; here every program comes from the compiler, because kernels are a fixed library."""

import numpy as np
import numpy.testing as npt
import pytest

from helpers import graph, node, ts

pytestmark = pytest.mark.gpu
F16 = "float16"


def run_program(ir, inputs_np, weights_np=None):
    from cuda_compiler import compile_subgraph
    from cuda_runtime import CUDABuffer, CUDAExecutor

    ex = CUDAExecutor(compile_subgraph(ir))
    ins = {k: CUDABuffer.from_numpy(v.astype(np.float16)) for k, v in inputs_np.items()}
    ws = {k: CUDABuffer.from_numpy(v.astype(np.float16)) for k, v in (weights_np or {}).items()}
    return {k: v.to_numpy().astype(np.float32) for k, v in ex.run(ins, ws).items()}, ex


def silu(x):
    return x / (1 + np.exp(-x.astype(np.float64)))


# ---- buffers and backend (test_cuda_executor.py:73-128) -------------------------------------
def test_buffer_round_trip_zeros_shape_and_write():
    from cuda_runtime import CUDABuffer

    data = np.random.RandomState(0).randn(4, 8).astype(np.float16)
    buf = CUDABuffer.from_numpy(data)
    npt.assert_array_equal(buf.to_numpy(), data)
    assert buf.shape == (4, 8) and buf.alloc_shape == (4, 8) and buf.size_bytes == 64 and buf.dtype == np.float16
    z = CUDABuffer.zeros((3, 5), np.dtype(np.float16))
    assert z.shape == (3, 5) and not z.to_numpy().any()
    new = np.random.RandomState(1).randn(3, 5).astype(np.float16)
    z.write_from_numpy(new)
    npt.assert_array_equal(z.to_numpy(), new)
    ids = np.array([[70000, 3]], dtype=np.int64)          # an fp16 buffer retyped by an integer write, exactly
    z.write_from_numpy(ids)
    npt.assert_array_equal(z.to_numpy(), ids)


def test_backend_name_allocate_and_synchronize():
    from cuda_runtime import CUDABackend, CUDABuffer
    from npu_runtime.backend import Backend, DeviceBuffer

    be = CUDABackend()
    assert be.name == "cuda" and isinstance(be, Backend)
    data = np.arange(12, dtype=np.float16).reshape(3, 4)
    buf = be.allocate_buffer(data)
    assert isinstance(buf, CUDABuffer) and isinstance(buf, DeviceBuffer)
    npt.assert_array_equal(buf.to_numpy(), data)
    z = be.allocate_zeros((2, 3))
    assert z.shape == (2, 3) and z.dtype == np.float16 and not z.to_numpy().any()
    be.synchronize()


# ---- single ops and fused chains -----------------------------------------------------------------
def unary(op, n=256):
    x, y = ts("x", [n], F16), ts("y", [n], F16)
    return graph([node(op.split(".")[1], op, [x], [y])], [x], [y])


def test_relu_and_neg():
    rs = np.random.RandomState(42)
    x = rs.randn(256).astype(np.float32)
    out, _ = run_program(unary("aten.relu.default"), {"x": x})
    npt.assert_allclose(out["y"], np.maximum(x.astype(np.float16), 0), rtol=1e-2, atol=1e-3)
    out, _ = run_program(unary("aten.neg.default"), {"x": x})
    npt.assert_allclose(out["y"], -x.astype(np.float16).astype(np.float32), rtol=1e-2, atol=1e-3)


def test_relu_add_and_add_relu_are_one_fused_step():
    from cuda_compiler.cuda_program import FusedKernelStep

    rs = np.random.RandomState(42)
    a, b = rs.randn(4, 64).astype(np.float32), rs.randn(4, 64).astype(np.float32)
    A, B = ts("a", [4, 64], F16), ts("b", [4, 64], F16)
    # relu(a) + b
    ir = graph([node("r", "aten.relu.default", [A], [ts("r", [4, 64], F16)]),
                node("y", "aten.add.Tensor", [ts("r", [4, 64], F16), B], [ts("y", [4, 64], F16)])], [A, B], [ts("y", [4, 64], F16)])
    out, ex = run_program(ir, {"a": a, "b": b})
    npt.assert_allclose(out["y"], np.maximum(a, 0) + b, rtol=1e-1, atol=1e-1)
    assert len([s for s in ex._program.steps if isinstance(s, FusedKernelStep)]) == 1
    # relu(a + b): the ResNet skip connection
    ir = graph([node("s", "aten.add.Tensor", [A, B], [ts("s", [4, 64], F16)]),
                node("y", "aten.relu.default", [ts("s", [4, 64], F16)], [ts("y", [4, 64], F16)])], [A, B], [ts("y", [4, 64], F16)])
    out, ex = run_program(ir, {"a": a, "b": b})
    npt.assert_allclose(out["y"], np.maximum(a + b, 0), rtol=1e-1, atol=1e-1)
    assert len([s for s in ex._program.steps if isinstance(s, FusedKernelStep)]) == 1


def test_silu_mul_fused():
    rs = np.random.RandomState(42)
    g, u = rs.randn(8, 128).astype(np.float32), rs.randn(8, 128).astype(np.float32)
    G, U = ts("gate", [8, 128], F16), ts("up", [8, 128], F16)
    ir = graph([node("s", "aten.silu.default", [G], [ts("s", [8, 128], F16)]),
                node("y", "aten.mul.Tensor", [ts("s", [8, 128], F16), U], [ts("y", [8, 128], F16)])], [G, U], [ts("y", [8, 128], F16)])
    out, _ = run_program(ir, {"gate": g, "up": u})
    npt.assert_allclose(out["y"], silu(g) * u, rtol=5e-2, atol=1e-2)


def test_gemm_and_linear_relu():
    rs = np.random.RandomState(42)
    x, w = rs.randn(1, 64).astype(np.float16), rs.randn(32, 64).astype(np.float16)
    X, W = ts("x", [1, 64], F16), ts("w", [32, 64], F16)
    ir = graph([node("y", "aten.linear.default", [X, W], [ts("y", [1, 32], F16)])], [X], [ts("y", [1, 32], F16)], [W])
    out, _ = run_program(ir, {"x": x}, {"w": w})
    want = x.astype(np.float32) @ w.astype(np.float32).T
    npt.assert_allclose(out["y"], want, rtol=5e-2, atol=5e-2)
    ir = graph([node("l", "aten.linear.default", [X, W], [ts("l", [1, 32], F16)]),
                node("y", "aten.relu.default", [ts("l", [1, 32], F16)], [ts("y", [1, 32], F16)])], [X], [ts("y", [1, 32], F16)], [W])
    out, _ = run_program(ir, {"x": x}, {"w": w})
    npt.assert_allclose(out["y"], np.maximum(want, 0), rtol=1e-1, atol=1e-1)


def test_reshape_is_exact_and_softmax():
    rs = np.random.RandomState(42)
    x = rs.randn(4, 64).astype(np.float16)
    X = ts("x", [4, 64], F16)
    ir = graph([node("r", "aten.reshape.default", [X], [ts("r", [8, 32], F16)], shape=[8, 32]),
                node("y", "aten.relu.default", [ts("r", [8, 32], F16)], [ts("y", [8, 32], F16)])], [X], [ts("y", [8, 32], F16)])
    out, _ = run_program(ir, {"x": x})
    npt.assert_array_equal(out["y"], np.maximum(x, 0).reshape(8, 32).astype(np.float32))
    ir = graph([node("y", "aten.softmax.int", [X], [ts("y", [4, 64], F16)], dim=-1)], [X], [ts("y", [4, 64], F16)])
    out, _ = run_program(ir, {"x": x})
    e = np.exp(x.astype(np.float64) - x.astype(np.float64).max(-1, keepdims=True))
    npt.assert_allclose(out["y"], e / e.sum(-1, keepdims=True), rtol=5e-2, atol=1e-2)
    npt.assert_allclose(out["y"].sum(-1), 1.0, atol=1e-2)


def test_tiny_gated_mlp():
    """gate/up/down projections with silu(gate) * up in between (test_cuda_fusion.py:293-374): hidden 64, inter 128."""
    rs = np.random.RandomState(42)
    H, I = 64, 128
    x = (rs.randn(1, H) * 0.5).astype(np.float32)
    wg, wu, wd = ((rs.randn(*s) * 0.1).astype(np.float32) for s in ((I, H), (I, H), (H, I)))
    X = ts("x", [1, H], F16)
    t = lambda n, s: ts(n, s, F16)
    ir = graph([node("g", "aten.linear.default", [X, t("wg", [I, H])], [t("g", [1, I])]),
                node("u", "aten.linear.default", [X, t("wu", [I, H])], [t("u", [1, I])]),
                node("s", "aten.silu.default", [t("g", [1, I])], [t("s", [1, I])]),
                node("m", "aten.mul.Tensor", [t("s", [1, I]), t("u", [1, I])], [t("m", [1, I])]),
                node("y", "aten.linear.default", [t("m", [1, I]), t("wd", [H, I])], [t("y", [1, H])])],
               [X], [t("y", [1, H])], [t("wg", [I, H]), t("wu", [I, H]), t("wd", [H, I])])
    out, _ = run_program(ir, {"x": x}, {"wg": wg, "wu": wu, "wd": wd})
    want = (silu(x @ wg.T) * (x @ wu.T)) @ wd.T
    npt.assert_allclose(out["y"], want, rtol=1e-1, atol=1e-1)
