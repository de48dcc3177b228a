"""CUDA runtime for B200: ``CUDABackend`` / ``CUDABuffer`` / ``CUDAExecutor``.

Importing this package never needs a GPU (mirrors the reference, whose
``cuda_runtime`` imports without CuPy - tests/test_extensibility.py:213-221);
constructing a backend or executor without one raises ``RuntimeError``.
"""

from cuda_runtime.cuda_backend import CUDABackend, CUDABuffer  # noqa: F401
from cuda_runtime.cuda_executor import CUDAExecutor  # noqa: F401
