"""Pins the CPU oracle: known-answer graphs of the reference's CPU-fallback tests
(tests/test_cpu_fallback.py:14-173) and eager-module golden fixtures."""

from pathlib import Path

import numpy as np
import numpy.testing as npt
import torch

import model_zoo as mz
from helpers import graph, node, ts
from ir_export import extract_ir
from oracle.ir_interpreter import IRInterpreter, execute_cpu_partition, numpy_to_torch, torch_to_numpy

GOLDEN = Path(__file__).parent / "golden"


def test_float32_roundtrip():
    arr = np.random.RandomState(0).randn(2, 3).astype(np.float32)
    t = numpy_to_torch(arr)
    assert t.dtype == torch.float32
    npt.assert_array_equal(arr, torch_to_numpy(t))


def test_bfloat16_roundtrip_is_bit_exact():
    t = torch.randn(2, 3, dtype=torch.bfloat16)
    arr = torch_to_numpy(t)
    assert arr.dtype.name == "bfloat16"
    back = numpy_to_torch(arr)
    assert back.dtype == torch.bfloat16
    npt.assert_array_equal(t.view(torch.uint16).numpy(), back.view(torch.uint16).numpy())


def test_known_answer_add():
    n = [node("add_node", "aten.add.Tensor", [ts("a", [2, 3]), ts("b", [2, 3])], [ts("c", [2, 3])])]
    a, b = np.full((2, 3), 2.0, np.float32), np.full((2, 3), 3.0, np.float32)
    out = execute_cpu_partition(n, {"a": a, "b": b}, weights={})
    npt.assert_allclose(out["c"], a + b)


def test_known_answer_relu():
    n = [node("relu_node", "aten.relu.default", [ts("x", [2, 4])], [ts("y", [2, 4])])]
    x = np.array([[-1, 2, -3, 4], [5, -6, 7, -8]], np.float32)
    npt.assert_allclose(execute_cpu_partition(n, {"x": x}, weights={})["y"], np.maximum(x, 0))


def test_known_answer_neg_relu_chain():
    n = [node("neg_node", "aten.neg.default", [ts("x", [2, 3])], [ts("neg_out", [2, 3])]),
         node("relu_node", "aten.relu.default", [ts("neg_out", [2, 3])], [ts("y", [2, 3])])]
    x = np.array([[-1, 2, -3], [4, -5, 6]], np.float32)
    npt.assert_allclose(execute_cpu_partition(n, {"x": x}, weights={})["y"], np.maximum(-x, 0))


def test_known_answer_mul_broadcast():
    n = [node("mul_node", "aten.mul.Tensor", [ts("x", [2, 3]), ts("scale", [1])], [ts("y", [2, 3])])]
    x = np.full((2, 3), 4.0, np.float32)
    out = execute_cpu_partition(n, {"x": x, "scale": np.array([2.0], np.float32)}, weights={})
    npt.assert_allclose(out["y"], x * 2.0)


def test_scalar_attr_operand():
    n = [node("m", "aten.mul.Tensor", [ts("x", [4])], [ts("y", [4])], other=0.5)]
    out = execute_cpu_partition(n, {"x": np.arange(4, dtype=np.float32)}, weights={})
    npt.assert_allclose(out["y"], np.arange(4) * 0.5)


def test_golden_resnet18():
    fx = np.load(GOLDEN / "resnet18_b2_64.npz")
    m = mz.resnet(18, seed=0)
    x = torch.from_numpy(fx["x"])
    ir = extract_ir(m, (x,), "resnet18")
    out = IRInterpreter(ir, m.state_dict()).execute({"x": x})
    npt.assert_array_equal(list(out.values())[0].numpy(), fx["logits"])


def test_golden_qwen_tiny_prefill_and_decode():
    from golden.make_golden import tiny_qwen

    fx = np.load(GOLDEN / "qwen_tiny.npz")
    cfg, sd, model = tiny_qwen()
    T, S = int(fx["T"]), int(fx["S"])
    L = cfg.num_hidden_layers
    ids = torch.from_numpy(fx["ids"])
    irp = extract_ir(mz.QwenPrefillWrapper(model), mz.qwen2_example_inputs(cfg, 1, T, None, device="cpu"), "p")
    pre = IRInterpreter(irp, sd).execute((ids, mz.causal_mask(1, T, T, 0), torch.arange(T)[None], torch.arange(T)))
    pre = list(pre.values())
    npt.assert_array_equal(pre[0].view(torch.uint16).numpy(), fx["prefill_logits"])
    npt.assert_array_equal(pre[1].contiguous().view(torch.uint16).numpy(), fx["prefill_k0"])
    kv = []
    for t in pre[1:]:
        buf = torch.zeros(1, t.shape[1], S, t.shape[3], dtype=torch.bfloat16)
        buf[:, :, :T] = t
        kv.append(buf)
    ird = extract_ir(mz.QwenDecodeWrapper(model, L), mz.qwen2_example_inputs(cfg, 1, 1, S, device="cpu"), "d")
    dec = IRInterpreter(ird, sd).execute((torch.from_numpy(fx["next_id"]), mz.causal_mask(1, 1, S, T), torch.tensor([[T]]),
                                           torch.tensor([T]), *kv))
    dec = list(dec.values())
    npt.assert_array_equal(dec[0].view(torch.uint16).numpy(), fx["decode_logits"])
    npt.assert_array_equal(dec[1].view(torch.uint16).numpy(), fx["decode_k0"])
