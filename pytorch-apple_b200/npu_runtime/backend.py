"""Abstract device interfaces every execution backend implements.

Method-for-method the contract of the reference ABCs
(npu_runtime/backend.py:11-68): a ``DeviceBuffer`` is a device allocation with
numpy interop, a ``Backend`` allocates buffers and runs compiled programs.
"""

from __future__ import annotations

from abc import ABC, abstractmethod
from typing import Any

import numpy as np


class DeviceBuffer(ABC):
    @property
    @abstractmethod
    def shape(self) -> tuple[int, ...]: ...

    @property
    @abstractmethod
    def alloc_shape(self) -> tuple[int, ...]: ...

    @property
    @abstractmethod
    def dtype(self) -> np.dtype: ...

    @property
    @abstractmethod
    def size_bytes(self) -> int: ...

    @property
    @abstractmethod
    def native_handle(self) -> Any:
        """The backend's own array object behind this buffer."""

    @abstractmethod
    def to_numpy(self, spec=None) -> np.ndarray: ...


class Backend(ABC):
    @property
    @abstractmethod
    def name(self) -> str: ...

    @property
    @abstractmethod
    def device(self) -> Any: ...

    @abstractmethod
    def allocate_buffer(self, data: np.ndarray, alloc_shape=None, spec=None) -> DeviceBuffer: ...

    @abstractmethod
    def allocate_zeros(self, shape, dtype=np.dtype(np.float16), alloc_shape=None) -> DeviceBuffer: ...

    @abstractmethod
    def execute(self, program, inputs, weights) -> dict[str, DeviceBuffer]: ...

    @abstractmethod
    def create_executor(self, program) -> Any:
        """Return an object with ``run(inputs, weights)`` that can be reused across calls."""

    @abstractmethod
    def synchronize(self): ...
