"""The reference's own ``DAGExecutor`` (unmodified source) driving this CUDA backend.

Needs the reference tree, which exists only where this repository was developed; elsewhere the
test is skipped (the GPU tests never read it).  The cases run in a child process because they
import ``npu_runtime`` / ``npu_compiler`` from the reference while the rest of the suite uses
this repository's mirrors of those modules."""

import os
import subprocess
import sys
from pathlib import Path

import pytest

REF = Path(os.environ.get("B200NN_REFERENCE_TREE", "/root/reference"))


@pytest.mark.skipif(not (REF / "npu_runtime" / "dag_executor.py").exists(), reason="reference tree not present")
def test_unmodified_reference_dag_executor_runs_on_this_backend():
    case = Path(__file__).with_name("reference_orchestrator_case.py")
    res = subprocess.run([sys.executable, str(case), str(REF), "fake"], capture_output=True, text=True, timeout=900)
    assert res.returncode == 0, res.stdout[-3000:] + res.stderr[-3000:]
    assert res.stdout.count("ok:") == 3, res.stdout


# The reference's own offline test files, unmodified, run against this repository's cuda_compiler /
# cuda_runtime / torch_ir (with the reference's npu_compiler / npu_runtime beside them).  Everything must
# pass except the cases below, which assert the reference's *fusion granularity or kernel source text*
# and fail because this compiler fuses more or emits no source strings:
EXPECTED_DEVIATIONS = {
    # relu after a linear layer rides in the GEMM epilogue here (the reference keeps a separate fused step)
    "test_cuda_compiler.py::TestSubgraphAnalyzer::test_blas_breaks_fusion",
    # the reference checks NVRTC source text (`__hmax`, `hexp`, `cuda_fp16.h`); there is no generated source, kernels are a fixed library
    "test_cuda_compiler.py::TestCUDACodegen::test_generate_relu_kernel",
    "test_cuda_compiler.py::TestCUDACodegen::test_generate_silu_mul_kernel",
    # conv + batch-norm + relu (+ residual add) collapse into one convolution step each: fewer fused steps than the reference counts
    "test_cuda_compiler.py::TestCompileSubgraph::test_resnet_basic_block",
    # gate and up projections share one GEMM with the silu(gate) * up epilogue: 2 GEMM steps instead of 3 + 1 fused
    "test_cuda_compiler.py::TestCompileSubgraph::test_qwen_mlp_pattern",
}


@pytest.mark.skipif(not (REF / "tests" / "test_cuda_compiler.py").exists(), reason="reference tree not present")
def test_reference_offline_tests_run_against_this_compiler(tmp_path):
    import shutil

    pkg = Path(__file__).resolve().parents[1] / "pytorch-apple_b200"
    for name, src in (("npu_runtime", REF / "npu_runtime"), ("npu_compiler", REF / "npu_compiler"), ("cuda_compiler", pkg / "cuda_compiler"),
                      ("cuda_runtime", pkg / "cuda_runtime"), ("torch_ir", pkg / "torch_ir"), ("ir_export.py", pkg / "ir_export.py")):
        os.symlink(src, tmp_path / name)
    tdir = tmp_path / "t"
    tdir.mkdir()
    files = ["test_cuda_compiler.py", "test_partitioner.py", "test_cpu_fallback.py", "test_extensibility.py"]
    for f in files:
        shutil.copy(REF / "tests" / f, tdir / f)
    env = dict(os.environ, PYTHONPATH=str(tmp_path))
    res = subprocess.run([sys.executable, "-m", "pytest", "-q", "--no-header", "-p", "no:cacheprovider", "-rf", "."], cwd=tdir, env=env,
                         capture_output=True, text=True, timeout=900)
    failed = {line.split()[1] for line in res.stdout.splitlines() if line.startswith("FAILED ")}
    assert failed == EXPECTED_DEVIATIONS, res.stdout[-3000:]
    tally = [line for line in res.stdout.splitlines() if " passed" in line][-1]
    assert int(tally.split(" passed")[0].split()[-1]) >= 66, tally
