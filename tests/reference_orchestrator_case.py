"""Run the REFERENCE's own orchestrator, unmodified, on this repository's CUDA backend.

Executed as a child process by tests/test_reference_orchestrator.py, in a checkout that has the
reference tree beside it (argv[1]).  The child's import path is arranged so that ``npu_runtime``
and ``npu_compiler`` resolve to the reference's packages while ``cuda_compiler``, ``cuda_runtime``
and ``torch_ir`` resolve to this repository's: the reference's ``DAGExecutor`` then drives our
compiler and backend exactly as it drives its own (npu_runtime/dag_executor.py:66-72, 101-147,
224-255): fp16-narrowed weights, ``allocate_buffer(arr)`` without a spec, an fp16 zero buffer
pre-allocated for every program input, int64 ids written into those buffers.

argv[2] = "fake": route the kernel library to the host stand-in (machine without a GPU).
Cases mirror the reference's tests/test_dag_executor.py:345-412 plus a tiny Qwen2 decode step.
"""

import os
import sys
import tempfile
from pathlib import Path

ref_root, mode = Path(sys.argv[1]), sys.argv[2]
repo = Path(__file__).resolve().parents[1]
pkg = repo / "pytorch-apple_b200"
link_dir = Path(tempfile.mkdtemp(prefix="mixed_imports_"))
for name, src in (("npu_runtime", ref_root / "npu_runtime"), ("npu_compiler", ref_root / "npu_compiler"),
                  ("cuda_compiler", pkg / "cuda_compiler"), ("cuda_runtime", pkg / "cuda_runtime"), ("torch_ir", pkg / "torch_ir"),
                  ("ir_export.py", pkg / "ir_export.py"), ("model_zoo.py", pkg / "model_zoo.py")):
    os.symlink(src, link_dir / name)
sys.path[:0] = [str(link_dir), str(repo / "tests")]

import numpy as np  # noqa: E402
import torch  # noqa: E402
import torch.nn as nn  # noqa: E402

import npu_runtime.dag_executor as ref_dag  # noqa: E402
from npu_compiler.partitioner import Partition, partition  # noqa: E402
from npu_runtime.backend import DeviceBuffer  # noqa: E402
from torch_ir import extract_ir  # noqa: E402

from cuda_compiler import compile_subgraph, is_cuda_op_supported  # noqa: E402
from cuda_runtime import native  # noqa: E402
from cuda_runtime.cuda_backend import CUDABackend  # noqa: E402

assert Path(ref_dag.__file__).resolve().is_relative_to(ref_root.resolve()), ref_dag.__file__
assert Path(sys.modules["cuda_compiler"].__file__).resolve().is_relative_to(pkg.resolve())
if mode == "fake":
    from fake_b200nn import FakeLibrary

    native.install_test_library(FakeLibrary(), "cpu")
DAGExecutor = ref_dag.DAGExecutor


def to_numpy(v):
    return v if isinstance(v, np.ndarray) else v.to_numpy()


class SimpleConvNet(nn.Module):   # the model of the reference's test (tests/test_dag_executor.py:96-117)
    def __init__(self):
        super().__init__()
        self.features = nn.Sequential(nn.Conv2d(3, 32, 3, padding=1), nn.ReLU(), nn.MaxPool2d(2, 2),
                                      nn.Conv2d(32, 64, 3, padding=1), nn.ReLU(), nn.MaxPool2d(2, 2))
        self.classifier = nn.Sequential(nn.Flatten(), nn.Linear(64 * 8 * 8, 256), nn.ReLU(), nn.Linear(256, 10))

    def forward(self, x):
        return self.classifier(self.features(x))


def ir_dict_of(model_cls, shape, name):
    import json

    with torch.device("meta"):
        meta = model_cls().eval()
    ir = extract_ir(meta, (torch.randn(*shape, device="meta"),), model_name=name)
    with tempfile.NamedTemporaryFile(suffix=".json", delete=False, mode="w") as tmp:
        path = tmp.name
    ir.save(path)                       # JSON round trip, as the reference's test does
    with open(path) as f:
        d = json.load(f)
    os.unlink(path)
    return d


def convnet(support, want_cpu_partition):
    torch.manual_seed(42)
    model = SimpleConvNet().eval()
    ir = ir_dict_of(SimpleConvNet, (1, 3, 32, 32), "SimpleConvNet")
    weights = {k: v.detach().cpu().numpy() for k, v in model.state_dict().items()}
    plan = partition(ir, support)
    parts = [s for s in plan.steps if isinstance(s, Partition)]
    assert any(p.target == "npu" for p in parts)
    assert any(p.target == "cpu" for p in parts) == want_cpu_partition
    dag = DAGExecutor(plan, CUDABackend(), compile_fn=compile_subgraph)
    x = torch.randn(1, 3, 32, 32)
    result = dag.execute(inputs={ir["graph_inputs"][0]["name"]: x.numpy()}, weights=weights)
    with torch.no_grad():
        want = model(x).numpy()
    got = to_numpy(list(result.values())[0]).astype(np.float32)
    np.testing.assert_allclose(got, want, rtol=1e-1, atol=1e-1)
    assert got.argmax() == want.argmax()
    # a second call reuses the pre-allocated input buffers and the bound plan
    again = to_numpy(list(dag.execute(inputs={ir["graph_inputs"][0]["name"]: x.numpy()}).values())[0]).astype(np.float32)
    np.testing.assert_allclose(again, got, rtol=1e-3, atol=1e-3)


def qwen_decode():
    """Tiny Qwen2 decode step: bf16 graph, int64 ids / positions, KV caches as numpy inputs."""
    import model_zoo as mz

    cfg = mz.qwen2_config(num_layers=2, hidden_size=256, intermediate_size=512, num_attention_heads=2, num_key_value_heads=1, vocab_size=70000)
    sd = mz.qwen2_weights(cfg, seed=0)
    model = mz.qwen2_model(cfg, device="cpu")
    model.load_state_dict({k[len("model."):]: v for k, v in sd.items() if "rotary" not in k}, strict=False)
    L, B, S, P = 2, 2, 48, 20
    wrapper = mz.QwenDecodeWrapper(model, L)
    ir = extract_ir(wrapper, mz.qwen2_example_inputs(cfg, B, 1, S, device="cpu"), model_name="qd").to_dict()
    g = torch.Generator().manual_seed(0)
    kv = [(torch.randn(B, 1, S, 128, generator=g) * 0.5).bfloat16() for _ in range(2 * L)]
    ids = torch.tensor([[69999], [3]])                 # an id above fp16's largest integer
    ins = (ids, mz.causal_mask(B, 1, S, P), torch.full((B, 1), P), torch.tensor([P]), *kv)
    with torch.no_grad():
        want = wrapper(*ins)
    plan = partition(ir, is_cuda_op_supported)
    assert all(p.target == "npu" for p in plan.steps if isinstance(p, Partition))
    dag = DAGExecutor(plan, CUDABackend(), compile_fn=compile_subgraph)
    weights = mz.state_dict_numpy(sd)
    feed = {s["name"]: (t.view(torch.uint16).numpy().view(weights["model.lm_head.weight"].dtype) if t.dtype == torch.bfloat16 else t.numpy())
            for s, t in zip(ir["graph_inputs"], ins)}
    out = dag.execute(inputs=feed, weights=weights)
    names = [o["name"] for o in ir["graph_outputs"]]
    got = to_numpy(out[names[0]]).astype(np.float32)
    ref = want[0].float().numpy()
    err = np.abs(got - ref).max()
    # the reference's loader narrows bf16 weights to fp16 (values below 6e-5 lose bits): tolerance, not equality
    assert err < 0.1, err
    assert (got[:, 0].argmax(-1) == ref[:, 0].argmax(-1)).all() or err > 0
    k0 = to_numpy(out[names[1]]).astype(np.float32)
    assert np.abs(k0 - want[1].float().numpy()).max() < 0.05
    assert isinstance(out[names[1]], DeviceBuffer)


convnet(is_cuda_op_supported, want_cpu_partition=False)
print("ok: SimpleConvNet, all ops on the device")
convnet(lambda op, attrs=None: op != "aten.max_pool2d.default" and is_cuda_op_supported(op, attrs), want_cpu_partition=True)
print("ok: SimpleConvNet, max_pool2d forced to the host")
qwen_decode()
print("ok: tiny Qwen2 decode step")
