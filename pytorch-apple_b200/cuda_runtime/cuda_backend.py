"""``Backend`` / ``DeviceBuffer`` implementations over ``torch`` device tensors.

Same classes, constructor arguments and methods as the reference backend
(cuda_runtime/cuda_backend.py:24-150), with ``torch.Tensor`` as the native handle
instead of ``cupy.ndarray``.  Differences that matter to callers:

* dtypes are preserved.  The reference coerces every non-integer upload to IEEE
  fp16 (cuda_backend.py:112-129, 78-91), which corrupts bfloat16 weights and token
  ids; here bf16 stays bf16 (numpy side: ``ml_dtypes.bfloat16`` or raw uint16),
  int64 stays int64, and float32 is narrowed only when a spec asks for fp16/bf16;
* ``write_from_numpy`` retypes the buffer from the spec/data, because the DAG
  executor pre-allocates every input as fp16 zeros (npu_runtime/dag_executor.py:108-116).
"""

from __future__ import annotations

from typing import Any

import numpy as np

from cuda_runtime import native
from npu_runtime.backend import Backend, DeviceBuffer

try:  # torch provides device memory and streams only
    import torch
except ImportError:  # pragma: no cover
    torch = None

_NP_TO_TORCH = {"float32": "float32", "float16": "float16", "int32": "int32", "int64": "int64", "uint8": "uint8",
                "bool": "bool", "float64": "float64", "int8": "int8", "int16": "int16"}


def _np_bf16():
    import ml_dtypes

    return np.dtype(ml_dtypes.bfloat16)


def _torch_dtype(name: str):
    return getattr(torch, name)


def numpy_to_torch(data: np.ndarray, target: str | None = None):
    """Host array -> host tensor.  bf16 arrives as ``ml_dtypes.bfloat16`` or uint16 bit
    patterns.  ``target`` (a torch dtype name) converts floats."""
    data = np.ascontiguousarray(data)
    if data.dtype.name == "bfloat16" or (data.dtype == np.uint16 and target == "bfloat16"):
        t = torch.from_numpy(data.view(np.uint16)).view(torch.bfloat16)
    elif data.dtype.name in _NP_TO_TORCH:
        t = torch.from_numpy(data)
    else:
        raise TypeError(f"unsupported numpy dtype {data.dtype}")
    if target is not None and t.dtype != _torch_dtype(target) and t.dtype.is_floating_point:
        t = t.to(_torch_dtype(target))
    return t


def torch_to_numpy(t) -> np.ndarray:
    """Host-side counterpart of ``numpy_to_torch``: a tensor as a numpy array, bfloat16 as an
    ``ml_dtypes.bfloat16`` view of the same bits (numpy has no native bfloat16)."""
    t = t.detach().cpu().contiguous()
    if t.dtype == torch.bfloat16:
        return t.view(torch.uint16).numpy().view(_np_bf16())
    return t.numpy()


class PinnedStaging:
    """Page-locked host buffers for the transfers at partition boundaries and for step inputs.

    The reference moves tensors between host and device partitions with ``cp.asarray`` /
    ``cp.asnumpy`` on pageable memory (cuda_backend.py:52-71, dag_executor.py:316-329).  Here uploads
    go host array -> pinned buffer -> device (asynchronous, DMA at full PCIe rate) and downloads come
    back through a pinned buffer as well.  One buffer per (dtype, element count), reused; a buffer is
    only rewritten after the copy that last read it has finished (an event per buffer)."""

    MIN_BYTES = 1 << 16   # smaller transfers are latency-bound either way
    MAX_BYTES = 64 << 20  # larger ones (whole weight matrices at load time) are not worth keeping a pinned twin for

    def __init__(self):
        self._up: dict[tuple, tuple[Any, Any]] = {}
        self._down: dict[tuple, Any] = {}
        self.uploads = self.downloads = 0

    def upload(self, host, dst) -> None:
        """dst (device tensor) <- host (CPU tensor of the same dtype / element count)."""
        nbytes = host.numel() * host.element_size()
        if not dst.is_cuda or nbytes < self.MIN_BYTES or nbytes > self.MAX_BYTES or host.is_pinned():
            dst.copy_(host.reshape(dst.shape), non_blocking=True)   # (a caller's own pinned array is copied straight from where it is)
            return
        key = (host.dtype, host.numel())
        entry = self._up.get(key)
        if entry is None:
            entry = (torch.empty(host.numel(), dtype=host.dtype).pin_memory(), torch.cuda.Event())
            self._up[key] = entry
        else:
            entry[1].synchronize()
        pinned, event = entry
        pinned.copy_(host.reshape(-1))
        dst.copy_(pinned.view(dst.shape), non_blocking=True)
        event.record()
        self.uploads += 1

    def download(self, src):
        """CPU tensor holding a copy of src (device tensor, contiguous)."""
        nbytes = src.numel() * src.element_size()
        if not src.is_cuda or nbytes < self.MIN_BYTES or nbytes > self.MAX_BYTES:
            return src.cpu()
        key = (src.dtype, src.numel())
        pinned = self._down.get(key)
        if pinned is None:
            pinned = torch.empty(src.numel(), dtype=src.dtype).pin_memory()
            self._down[key] = pinned
        pinned.copy_(src.reshape(-1), non_blocking=True)
        torch.cuda.current_stream().synchronize()
        self.downloads += 1
        return pinned.view(src.shape).clone()


_staging: PinnedStaging | None = None


def staging() -> PinnedStaging:
    global _staging
    if _staging is None:
        _staging = PinnedStaging()
    return _staging


def _target_dtype(data: np.ndarray, spec) -> str | None:
    """Which dtype an upload should have on the device."""
    name = getattr(spec, "dtype", None) if spec is not None else None
    if data.dtype.kind in "iub":
        return None  # integers and bools are kept as they are
    if name in ("float16", "bfloat16"):
        return name
    return None  # float32 specs keep the host precision; the executor narrows on device


class CUDABuffer(DeviceBuffer):
    def __init__(self, data, logical_shape: tuple[int, ...] | None = None):
        self._data = data
        self._logical_shape = tuple(logical_shape) if logical_shape is not None else tuple(data.shape)

    @property
    def shape(self) -> tuple[int, ...]:
        return self._logical_shape

    @property
    def alloc_shape(self) -> tuple[int, ...]:
        return tuple(self._data.shape)

    @property
    def dtype(self) -> np.dtype:
        if self._data.dtype == torch.bfloat16:
            return _np_bf16()
        return np.dtype(str(self._data.dtype).replace("torch.", ""))

    @property
    def size_bytes(self) -> int:
        return self._data.numel() * self._data.element_size()

    @property
    def native_handle(self) -> Any:
        """The ``torch.Tensor`` on the device."""
        return self._data

    def to_numpy(self, spec=None, dtype=None) -> np.ndarray:
        t = self._data.detach()
        if not t.is_contiguous():
            t = t.contiguous()
        t = staging().download(t) if t.is_cuda else t.cpu()
        if t.dtype == torch.bfloat16:
            arr = t.view(torch.uint16).numpy().view(_np_bf16())
        else:
            arr = t.numpy()
        if tuple(arr.shape) != self._logical_shape:
            n = int(np.prod(self._logical_shape)) if self._logical_shape else 1
            arr = arr.reshape(-1)[:n].reshape(self._logical_shape)
        if dtype is not None and arr.dtype != np.dtype(dtype):
            arr = arr.astype(dtype)
        return arr

    @classmethod
    def from_numpy(cls, data: np.ndarray, dtype=None, device: str | None = None) -> "CUDABuffer":
        target = None
        if dtype is not None:
            target = "bfloat16" if getattr(np.dtype(dtype), "name", "") == "bfloat16" else np.dtype(dtype).name
        host = numpy_to_torch(data, target)
        dev = torch.empty(host.shape, dtype=host.dtype, device=device or native.device_string())
        staging().upload(host, dev)
        return cls(dev)

    @classmethod
    def zeros(cls, shape: tuple[int, ...], dtype=np.dtype(np.float16), device: str | None = None) -> "CUDABuffer":
        name = "bfloat16" if getattr(np.dtype(dtype), "name", "") == "bfloat16" else np.dtype(dtype).name
        return cls(torch.zeros(tuple(shape), dtype=_torch_dtype(name), device=device or native.device_string()))

    def write_from_numpy(self, data: np.ndarray, spec=None) -> None:
        host = numpy_to_torch(data, _target_dtype(data, spec))
        if host.dtype != self._data.dtype or tuple(host.shape) != tuple(self._data.shape):
            # first write after the fp16-zeros pre-allocation: adopt the real dtype/shape
            self._data = torch.empty(tuple(host.shape), dtype=host.dtype, device=self._data.device)
        staging().upload(host, self._data)
        self._logical_shape = tuple(data.shape)


class CUDABackend(Backend):
    def __init__(self, device_id: int = 0):
        if torch is None:
            raise RuntimeError("PyTorch is not installed; it provides device memory for the CUDA backend")
        native.load()  # RuntimeError if the kernel library is missing
        self._device_id = device_id
        self._device = native.device_string(device_id)
        if self._device.startswith("cuda"):
            if not torch.cuda.is_available():
                raise RuntimeError("no CUDA device is available")
            torch.cuda.set_device(device_id)

    @property
    def name(self) -> str:
        return "cuda"

    @property
    def device(self) -> Any:
        return torch.device(self._device)

    def allocate_buffer(self, data: np.ndarray, alloc_shape=None, spec=None) -> CUDABuffer:
        host = numpy_to_torch(data, _target_dtype(np.asarray(data), spec))
        dev = torch.empty(host.shape, dtype=host.dtype, device=self._device)
        staging().upload(host, dev)
        return CUDABuffer(dev)

    def allocate_zeros(self, shape, dtype=np.dtype(np.float16), alloc_shape=None) -> CUDABuffer:
        return CUDABuffer.zeros(tuple(shape), dtype=dtype, device=self._device)

    def execute(self, program, inputs, weights) -> dict[str, CUDABuffer]:
        return self.create_executor(program).run(inputs, weights)

    def create_executor(self, program) -> Any:
        from cuda_runtime.cuda_executor import CUDAExecutor

        return CUDAExecutor(program, device_id=self._device_id)

    def synchronize(self):
        if self._device.startswith("cuda"):
            torch.cuda.synchronize(self._device_id)
