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
