"""The shared library builds, loads, and exports exactly what include/b200nn.h declares.
No compute call is made here (no GPU)."""

import re
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parents[1]


def declared_symbols():
    text = (ROOT / "include" / "b200nn.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(b200_[a-z0-9_]+)\s*\(", text)))


def test_header_and_binding_agree():
    from cuda_runtime import native

    assert declared_symbols() == sorted(native.SIGNATURES)


def test_library_exports_every_declared_symbol(native_lib):
    for name in declared_symbols():
        assert hasattr(native_lib, name), name
    assert native_lib.b200_version() == 1


def test_host_only_entry_points(native_lib):
    # workspace sizing is pure host arithmetic
    assert native_lib.b200_linear_workspace_bytes(1, 1536, 1536) > 0
    assert native_lib.b200_linear_workspace_bytes(512, 1536, 1536) == 0
    assert native_lib.b200_attn_decode_workspace_bytes(64, 12, 2, 4352, 128) == 0   # the splits merge inside the kernel
    assert native_lib.b200_attn_decode_workspace_bytes(64, 12, 2, 8192, 128) == 0      # up to 16384 rows likewise
    assert native_lib.b200_attn_decode_workspace_bytes(64, 12, 2, 32768, 128) == 64 * 2 * 64 * 6 * 130 * 4   # longer caches: 512-key splits + merge kernel


def test_compiler_and_library_agree_on_the_splitk_shapes(native_lib):
    """The compiler appends an RMSNorm to a GEMM only for the shapes it expects the library to split over CTA pairs
    (`_pair_splitk_shape` of the lowering pass).  The library's own rule shows in its workspace sizing: for rows > 64 a
    non-zero size means exactly that path.  The two are kept in step here (a mismatch would not be wrong, only a
    fusion promised and not delivered, or missed)."""
    from cuda_compiler.subgraph_analyzer import _Lowering as SubgraphAnalyzer

    for M in (65, 128, 129, 256, 300, 512, 1000, 1024, 2048, 4096):
        for N in (256, 1024, 1200, 1536, 2048, 2056, 4096):
            for K in (1536, 4096, 4104, 8960):
                mirror = SubgraphAnalyzer._pair_splitk_shape(M, N, K)
                lib_splits = native_lib.b200_linear_workspace_bytes(M, N, K) > 0
                if mirror:
                    assert lib_splits, (M, N, K)
                elif lib_splits:   # shapes the library splits but whose rows it cannot normalise in the reduce kernel
                    assert N > 2048 or N % 8, (M, N, K)
    assert SubgraphAnalyzer._pair_splitk_shape(512, 1536, 8960) and SubgraphAnalyzer._pair_splitk_shape(1024, 1536, 8960)
    assert not SubgraphAnalyzer._pair_splitk_shape(2048, 1536, 8960) and not SubgraphAnalyzer._pair_splitk_shape(512, 1536, 1536)


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    from cuda_runtime import native

    monkeypatch.setenv("B200NN_LIBRARY", str(tmp_path / "nope.so"))
    monkeypatch.setattr(native, "_lib", None)
    with pytest.raises(RuntimeError, match="no fallback"):
        native.load()


def test_backend_without_gpu_raises_runtime_error(native_lib):
    import torch

    from cuda_runtime import CUDABackend, CUDABuffer
    from npu_runtime.backend import Backend, DeviceBuffer

    assert issubclass(CUDABackend, Backend) and issubclass(CUDABuffer, DeviceBuffer)
    if not torch.cuda.is_available():
        with pytest.raises(RuntimeError):
            CUDABackend()


def test_buffer_semantics_on_the_cpu_seam(fake_native):
    import ml_dtypes

    from cuda_runtime import CUDABackend, CUDABuffer
    from npu_compiler import TensorSpec

    be = CUDABackend()
    assert be.name == "cuda"
    a = np.arange(12, dtype=np.float32).reshape(3, 4)
    buf = be.allocate_buffer(a)
    assert buf.shape == (3, 4) and buf.dtype == np.float32 and buf.size_bytes == 48
    np.testing.assert_array_equal(buf.to_numpy(), a)
    z = be.allocate_zeros((2, 5))
    assert z.dtype == np.float16 and not z.to_numpy().any()
    # the DAG executor pre-allocates fp16 zeros for every input, ids included: writes must retype
    ids = np.array([[151935, 70000]], dtype=np.int64)
    z.write_from_numpy(ids, spec=TensorSpec("input_ids", [1, 2], "int64"))
    assert z.dtype == np.int64 and z.shape == (1, 2)
    np.testing.assert_array_equal(z.to_numpy(), ids)
    # bf16 travels as bit patterns
    b = np.array([1.0, 3.0e-6, -2.5], dtype=ml_dtypes.bfloat16)
    bb = CUDABuffer.from_numpy(b)
    assert bb.dtype == ml_dtypes.bfloat16
    np.testing.assert_array_equal(bb.to_numpy().view(np.uint16), b.view(np.uint16))
    np.testing.assert_array_equal(bb.to_numpy(dtype=np.float32), b.astype(np.float32))
    be.synchronize()
