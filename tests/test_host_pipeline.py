"""Whole host pipeline on CPU: IR -> patterns -> lowering -> arena -> argument binding
-> outputs, with the native library replaced by the torch stand-in
(tests/fake_b200nn.py) and the oracle as the checker.  These tests prove the host
logic (views, offsets, strides, operand order), not the CUDA kernels."""

from pathlib import Path

import numpy as np
import pytest
import torch

import model_zoo as mz
from helpers import graph, masked_softmax_graph, node, np_inputs, rmsnorm_graph, rope_graph, run_backend, silu_mul_graph, to_f32, ts
from ir_export import extract_ir
from oracle.ir_interpreter import IRInterpreter, cpu_executor_factory, torch_to_numpy

GOLDEN = Path(__file__).parent / "golden"


def oracle(ir, weights, inputs):
    return {k: to_f32(v) for k, v in IRInterpreter(ir, weights).execute(inputs).items()}


def assert_bf16_close(got, gold_bits, max_fraction=0.01):
    """bf16 results of a floating-point path: at most one unit in the last place, on few elements."""
    a = got.view(np.uint16).astype(np.int32)
    b = np.asarray(gold_bits).astype(np.int32)
    diff = np.abs(a - b)
    assert diff.max() <= 1 and (diff != 0).mean() <= max_fraction, (diff.max(), (diff != 0).mean())


def rand(shape, dtype=torch.bfloat16, seed=0, scale=1.0):
    return (torch.randn(*shape, generator=torch.Generator().manual_seed(seed)) * scale).to(dtype)


@pytest.mark.parametrize("rows", [1, 5, 128])
def test_rmsnorm_graph(fake_native, rows):
    ir = rmsnorm_graph(rows, 1536)
    x, w = rand((rows, 1536)), (1 + 0.02 * rand((1536,), seed=1).float()).bfloat16()
    out, _ = run_backend(ir, {"w": torch_to_numpy(w)}, {"x": torch_to_numpy(x)})
    ref = oracle(ir, {"w": w}, {"x": x})
    np.testing.assert_allclose(to_f32(out["y"]), ref["y"], rtol=2e-2, atol=1e-2)
    assert fake_native.calls == ["rmsnorm"]


def _linear_residual_rmsnorm_graph(M, N, K, dtype="bfloat16", eps=1e-6):
    """h = a @ W^T + r;  y = rmsnorm(h) * g  - the down projection of a layer and the next layer's input norm."""
    f32 = "float32"
    a, r, w, g = ts("a", [M, K], dtype), ts("r", [M, N], dtype), ts("w_down", [N, K], dtype), ts("g", [N], dtype)
    t = lambda n, d=dtype, c=N: ts(n, [M, c], d)
    n = [node("lin", "aten.linear.default", [a, w], [t("lin")]),
         node("h", "aten.add.Tensor", [r, t("lin")], [t("h")]),
         node("to_a", "aten.to.dtype", [t("h")], [t("to_a", f32)], dtype="torch.float32"),
         node("pow_1", "aten.pow.Tensor_Scalar", [t("to_a", f32)], [t("pow_1", f32)], exponent=2),
         node("mean", "aten.mean.dim", [t("pow_1", f32)], [t("mean", f32, 1)], dim=[-1], keepdim=True),
         node("add", "aten.add.Tensor", [t("mean", f32, 1)], [t("add", f32, 1)], other=eps),
         node("rsqrt", "aten.rsqrt.default", [t("add", f32, 1)], [t("rsqrt", f32, 1)]),
         node("mul_a", "aten.mul.Tensor", [t("to_a", f32), t("rsqrt", f32, 1)], [t("mul_a", f32)]),
         node("to_b", "aten.to.dtype", [t("mul_a", f32)], [t("to_b")], dtype="torch." + dtype),
         node("y", "aten.mul.Tensor", [g, t("to_b")], [t("y")])]
    return graph(n, [a, r], [t("h"), t("y")], [w, g])


def test_rmsnorm_rides_on_the_splitk_reduction_of_a_prefill_down_projection(fake_native):
    M, N, K = 512, 1536, 4096   # 12 tiles of 256 x 256, long reduction: the shape class the library splits over CTA pairs
    ir = _linear_residual_rmsnorm_graph(M, N, K)
    a, r = rand((M, K)), rand((M, N), seed=1)
    w, g = (0.02 * rand((N, K), seed=2).float()).bfloat16(), (1 + 0.02 * rand((N,), seed=3).float()).bfloat16()
    out, _ = run_backend(ir, {"w_down": torch_to_numpy(w), "g": torch_to_numpy(g)}, {"a": torch_to_numpy(a), "r": torch_to_numpy(r)})
    ref = oracle(ir, {"w_down": w, "g": g}, {"a": a, "r": r})
    np.testing.assert_allclose(to_f32(out["h"]), ref["h"], rtol=2e-2, atol=2e-2)
    np.testing.assert_allclose(to_f32(out["y"]), ref["y"], rtol=2e-2, atol=2e-2)
    assert fake_native.calls == ["linear_rmsnorm"]
    # a shape the library does not split keeps the two steps
    fake_native.calls.clear()
    ir2 = _linear_residual_rmsnorm_graph(128, 1536, 4096)
    run_backend(ir2, {"w_down": torch_to_numpy(w), "g": torch_to_numpy(g)}, {"a": torch_to_numpy(a[:128]), "r": torch_to_numpy(r[:128])})
    assert fake_native.calls == ["linear", "rmsnorm"]


def test_silu_mul_graph(fake_native):
    ir = silu_mul_graph(7, 8960)
    g, u = rand((7, 8960)), rand((7, 8960), seed=1)
    out, _ = run_backend(ir, {}, {"gate": torch_to_numpy(g), "up": torch_to_numpy(u)})
    np.testing.assert_allclose(to_f32(out["y"]), oracle(ir, {}, {"gate": g, "up": u})["y"], rtol=2e-2, atol=1e-2)


def test_masked_softmax_graph(fake_native):
    T = 40
    ir = masked_softmax_graph(12, T)
    s, m = rand((1, 12, T, T)), mz.causal_mask(1, T, T, 0)
    out, _ = run_backend(ir, {}, {"scores": torch_to_numpy(s), "mask": torch_to_numpy(m)})
    np.testing.assert_allclose(to_f32(out["y"]), oracle(ir, {}, {"scores": s, "mask": m})["y"], rtol=2e-2, atol=2e-3)
    assert fake_native.calls == ["softmax"]


def test_rope_graph(fake_native):
    T = 24
    ir = rope_graph(12, T)
    x = rand((1, 12, T, 128))
    pos = torch.arange(T)[None] + 1000
    inv = 1.0 / (1e6 ** (torch.arange(0, 128, 2).float() / 128))
    out, _ = run_backend(ir, {"inv_freq": inv.numpy()}, {"x": torch_to_numpy(x), "position_ids": pos.numpy()})
    ref = oracle(ir, {"inv_freq": inv}, {"x": x, "position_ids": pos})
    np.testing.assert_allclose(to_f32(out["y"]), ref["y"], rtol=2e-2, atol=2e-2)
    assert fake_native.calls == ["rope_table", "rope_rotate"]


def test_unfused_lowering_matches_too(fake_native):
    """fuse=False exercises the generic per-op path (views, chains, strided copies)."""
    T = 8
    ir = rope_graph(4, T)
    x = rand((1, 4, T, 128))
    pos = torch.arange(T)[None]
    inv = 1.0 / (1e6 ** (torch.arange(0, 128, 2).float() / 128))
    out, _ = run_backend(ir, {"inv_freq": inv.numpy()}, {"x": torch_to_numpy(x), "position_ids": pos.numpy()}, {"fuse": False})
    ref = oracle(ir, {"inv_freq": inv}, {"x": x, "position_ids": pos})
    np.testing.assert_allclose(to_f32(out["y"]), ref["y"], rtol=2e-2, atol=2e-2)
    assert "rope_rotate" not in fake_native.calls and "strided_copy" in fake_native.calls


def test_embedding_and_index_copy_are_bit_exact(fake_native):
    V, D, S = 300, 64, 16
    n = [node("emb", "aten.embedding.default", [ts("table", [V, D], "bfloat16"), ts("ids", [2, 3], "int64")], [ts("emb", [2, 3, D], "bfloat16")]),
         node("ic", "aten.index_copy.default", [ts("cache", [2, 2, S, D], "bfloat16"), ts("pos", [1], "int64"), ts("src", [2, 2, 1, D], "bfloat16")],
              [ts("ic", [2, 2, S, D], "bfloat16")], dim=2)]
    ir = graph(n, [ts("ids", [2, 3], "int64"), ts("cache", [2, 2, S, D], "bfloat16"), ts("pos", [1], "int64"), ts("src", [2, 2, 1, D], "bfloat16")],
               [ts("emb", [2, 3, D], "bfloat16"), ts("ic", [2, 2, S, D], "bfloat16")], [ts("table", [V, D], "bfloat16")])
    table, cache, src = rand((V, D)), rand((2, 2, S, D), seed=1), rand((2, 2, 1, D), seed=2)
    ids, pos = torch.tensor([[0, 299, 7], [151, 151, 2]]), torch.tensor([5])
    ins = {"ids": ids.numpy(), "cache": torch_to_numpy(cache), "pos": pos.numpy(), "src": torch_to_numpy(src)}
    out, _ = run_backend(ir, {"table": torch_to_numpy(table)}, ins)
    ref = IRInterpreter(ir, {"table": table}).execute({"ids": ids, "cache": cache, "pos": pos, "src": src})
    for k in ("emb", "ic"):
        np.testing.assert_array_equal(out[k].view(np.uint16), ref[k].view(torch.uint16).numpy())


def test_resnet18_golden(fake_native):
    fx = np.load(GOLDEN / "resnet18_b2_64.npz")
    m = mz.resnet(18, seed=0)
    ir = extract_ir(m, (torch.from_numpy(fx["x"]),), "resnet18")
    out, dag = run_backend(ir, mz.state_dict_numpy(m.state_dict()), {"x": fx["x"]})
    got = to_f32(out[ir["graph_outputs"][0]["name"]])
    np.testing.assert_allclose(got, fx["logits"], rtol=0, atol=1e-1)  # the reference's ResNet-18 tolerance
    assert (np.argsort(-got, 1)[:, :5] == np.argsort(-fx["logits"], 1)[:, :5]).all()
    assert fake_native.calls.count("conv2d") == 20 and "batch_norm" not in fake_native.calls


def test_qwen_tiny_golden_prefill_then_decode(fake_native):
    from golden.make_golden import tiny_qwen

    fx = np.load(GOLDEN / "qwen_tiny.npz")
    cfg, sd, model = tiny_qwen()
    T, S, L = int(fx["T"]), int(fx["S"]), cfg.num_hidden_layers
    w = mz.state_dict_numpy(sd)
    irp = extract_ir(mz.QwenPrefillWrapper(model), mz.qwen2_example_inputs(cfg, 1, T, None, device="cpu"), "p")
    ins = np_inputs(irp, (torch.from_numpy(fx["ids"]), mz.causal_mask(1, T, T, 0), torch.arange(T)[None], torch.arange(T)))
    pre, _ = run_backend(irp, w, ins)
    assert fake_native.calls.count("rope_rotate_pair") == L and "rope_rotate" not in fake_native.calls
    names = [o["name"] for o in irp["graph_outputs"]]
    gold = torch.from_numpy(fx["prefill_logits"]).view(torch.bfloat16).float().numpy()
    got = to_f32(pre[names[0]])
    assert np.abs(got - gold).max() < 0.1
    assert (got[0, -1].argmax() == gold[0, -1].argmax())
    assert_bf16_close(pre[names[1]], fx["prefill_k0"])  # K of layer 0: norm + GEMM + rope, last-bit differences only
    # decode on top of the prefilled cache
    kv = []
    for n in names[1:]:
        buf = np.zeros((1, 1, S, 128), dtype=pre[n].dtype)
        buf[:, :, :T] = pre[n]
        kv.append(buf)
    ird = extract_ir(mz.QwenDecodeWrapper(model, L), mz.qwen2_example_inputs(cfg, 1, 1, S, device="cpu"), "d")
    dins = dict(zip([s["name"] for s in ird["graph_inputs"]],
                    [fx["next_id"], torch_to_numpy(mz.causal_mask(1, 1, S, T)), np.array([[T]]), np.array([T])] + kv))
    dec, _ = run_backend(ird, w, dins)
    dn = [o["name"] for o in ird["graph_outputs"]]
    gold = torch.from_numpy(fx["decode_logits"]).view(torch.bfloat16).float().numpy()
    got = to_f32(dec[dn[0]])
    assert np.abs(got - gold).max() < 0.1 and got.argmax() == gold.argmax()
    assert_bf16_close(dec[dn[1]], fx["decode_k0"])
    assert fake_native.calls.count("attn_decode") == L and fake_native.calls.count("attn_prefill") == L


def test_mixed_partitions_use_the_injected_cpu_executor(fake_native):
    from cuda_compiler import compile_subgraph
    from cuda_runtime import CUDABackend
    from npu_compiler import partition
    from npu_runtime import DAGExecutor

    n = [node("a", "aten.relu.default", [ts("x", [2, 8])], [ts("a", [2, 8])]),
         node("b", "aten.neg.default", [ts("a", [2, 8])], [ts("b", [2, 8])]),
         node("c", "aten.add.Tensor", [ts("b", [2, 8]), ts("a", [2, 8])], [ts("c", [2, 8])])]
    ir = graph(n, [ts("x", [2, 8])], [ts("c", [2, 8])])
    plan = partition(ir, lambda op, attrs=None: op != "aten.neg.default")
    dag = DAGExecutor(plan, CUDABackend(), compile_subgraph, cpu_executor_factory=cpu_executor_factory)
    x = np.random.RandomState(0).randn(2, 8).astype(np.float32)
    out = dag.execute({"x": x}, weights={})
    c = out["c"] if isinstance(out["c"], np.ndarray) else out["c"].to_numpy()
    np.testing.assert_allclose(c.astype(np.float32), np.zeros((2, 8)), atol=1e-3)  # relu(x) - relu(x)


def test_cpu_partition_without_interpreter_raises(fake_native):
    from cuda_compiler import compile_subgraph
    from cuda_runtime import CUDABackend
    from npu_compiler import partition
    from npu_runtime import DAGExecutor

    ir = graph([node("b", "aten.neg.default", [ts("x", [2])], [ts("b", [2])])], [ts("x", [2])], [ts("b", [2])])
    dag = DAGExecutor(partition(ir, lambda *a: False), CUDABackend(), compile_subgraph)
    with pytest.raises(RuntimeError, match="torch_ir"):
        dag.execute({"x": np.zeros(2, np.float32)}, weights={})


def test_replacing_one_weight_buffer_in_the_same_dict_is_noticed(fake_native):
    """The executor keeps prepared copies and bound pointers per weight set; swapping one buffer
    inside the dict it was given (same dict object, same length) must rebuild them."""
    from cuda_compiler import compile_subgraph
    from cuda_runtime import CUDABackend

    n = [node("y", "aten.linear.default", [ts("x", [2, 8], "bfloat16"), ts("w", [4, 8], "bfloat16")], [ts("y", [2, 4], "bfloat16")])]
    ir = graph(n, [ts("x", [2, 8], "bfloat16")], [ts("y", [2, 4], "bfloat16")], [ts("w", [4, 8], "bfloat16")])
    backend = CUDABackend()
    ex = backend.create_executor(compile_subgraph(ir))
    x, w1, w2 = rand((2, 8)), rand((4, 8), seed=1), rand((4, 8), seed=2)
    weights = {"w": backend.allocate_buffer(torch_to_numpy(w1))}
    feed = {"x": backend.allocate_buffer(torch_to_numpy(x))}
    y1 = to_f32(ex.run(feed, weights)["y"])
    np.testing.assert_allclose(y1, (x.float() @ w1.float().T).numpy(), rtol=2e-2, atol=2e-2)
    weights["w"] = backend.allocate_buffer(torch_to_numpy(w2))      # same dict, one entry replaced
    y2 = to_f32(ex.run(feed, weights)["y"])
    np.testing.assert_allclose(y2, (x.float() @ w2.float().T).numpy(), rtol=2e-2, atol=2e-2)
    assert np.abs(y2 - y1).max() > 0.1


def test_cache_read_by_a_later_partition_is_not_updated_in_place(fake_native):
    """index_copy into a graph input is normally done in the caller's buffer.  When another partition of
    the plan reads the same input afterwards it must still see the old contents, as with the reference's
    out-of-place kernel (cuda_templates.py:134-162)."""
    from cuda_compiler import compile_subgraph
    from cuda_runtime import CUDABackend
    from npu_compiler import partition
    from npu_runtime import DAGExecutor

    S, D = 8, 16
    c, src, pos = ts("cache", [1, 1, S, D], "bfloat16"), ts("src", [1, 1, 1, D], "bfloat16"), ts("pos", [1], "int64")
    n = [node("upd", "aten.index_copy.default", [c, pos, src], [ts("upd", [1, 1, S, D], "bfloat16")], dim=2),
         node("old", "aten.neg.default", [c], [ts("old", [1, 1, S, D], "bfloat16")]),           # forced to the host: reads the cache after the update
         node("sum", "aten.add.Tensor", [ts("upd", [1, 1, S, D], "bfloat16"), ts("old", [1, 1, S, D], "bfloat16")], [ts("sum", [1, 1, S, D], "bfloat16")])]
    ir = graph(n, [c, pos, src], [ts("sum", [1, 1, S, D], "bfloat16"), ts("upd", [1, 1, S, D], "bfloat16")])
    plan = partition(ir, lambda op, attrs=None: op != "aten.neg.default")
    dag = DAGExecutor(plan, CUDABackend(), compile_subgraph, cpu_executor_factory=cpu_executor_factory)
    first = next(iter(dag.npu_programs.values()))
    assert not first.donated_inputs
    cache, row = rand((1, 1, S, D)), rand((1, 1, 1, D), seed=1)
    feed = {"cache": torch_to_numpy(cache), "pos": np.array([3]), "src": torch_to_numpy(row)}
    out = dag.execute(feed, weights={})
    ref = oracle(ir, {}, {"cache": cache, "pos": torch.tensor([3]), "src": row})
    np.testing.assert_allclose(to_f32(out["sum"]), ref["sum"], rtol=0, atol=1e-6)
    # alone in its plan the same update is done in place
    solo = graph(n[:1], [c, pos, src], [ts("upd", [1, 1, S, D], "bfloat16")])
    assert compile_subgraph(solo).donated_inputs == {"upd": "cache"}
    assert not compile_subgraph(solo, keep_inputs={"cache"}).donated_inputs


def test_program_save_and_load_round_trip(fake_native, tmp_path):
    """A compiled program written to disk and read back drives the executor to the same result
    (the reference has save / load for its Metal programs only, npu_compiler/compiled_program.py:49-117)."""
    from golden.make_golden import tiny_qwen

    from cuda_compiler import compile_subgraph
    from cuda_compiler.cuda_program import CUDAProgram
    from cuda_runtime import CUDABackend

    cfg, sd, model = tiny_qwen()
    L, B, S, P = cfg.num_hidden_layers, 2, 40, 17
    ir = extract_ir(mz.QwenDecodeWrapper(model, L), mz.qwen2_example_inputs(cfg, B, 1, S, device="cpu"), "d")
    prog = compile_subgraph(ir)
    path = tmp_path / "decode.b200prog"
    prog.save(str(path))
    back = CUDAProgram.load(str(path))
    assert back.to_dict() == prog.to_dict()
    assert type(back.steps[0]) is type(prog.steps[0]) and back.views.keys() == prog.views.keys()
    assert [a.offset for a in back.buffer_allocations] == [a.offset for a in prog.buffer_allocations] and back.arena_bytes == prog.arena_bytes
    g = torch.Generator().manual_seed(2)
    ins = (torch.randint(0, cfg.vocab_size, (B, 1), generator=g), mz.causal_mask(B, 1, S, P), torch.full((B, 1), P), torch.tensor([P]),
           *[(torch.randn(B, 1, S, 128, generator=g) * 0.5).bfloat16() for _ in range(2 * L)])
    backend = CUDABackend()
    w = mz.state_dict_numpy(sd)
    outs = []
    for program in (prog, back):
        ex = backend.create_executor(program)
        key_to_ph = {k: ph for ph, k in program.weight_name_mapping.items()}
        weights = {key_to_ph.get(s.name, s.name): backend.allocate_buffer(w[s.name], spec=s) for s in program.weight_specs if s.name in w}
        feed = {s["name"]: backend.allocate_buffer(torch_to_numpy(t)) for s, t in zip(ir["graph_inputs"], ins)}
        outs.append(to_f32(ex.run(feed, weights)[ir["graph_outputs"][0]["name"]]))
    np.testing.assert_array_equal(outs[0], outs[1])
    ref = oracle(ir, sd, ins)[ir["graph_outputs"][0]["name"]]
    assert np.abs(outs[1] - ref).max() < 0.1
    with pytest.raises(ValueError, match="version"):
        CUDAProgram.from_dict({**prog.to_dict(), "version": 99})
