"""Runtime-side boundary: the backend ABCs and the partition orchestrator."""

from npu_runtime.backend import Backend, DeviceBuffer  # noqa: F401
from npu_runtime.dag_executor import DAGExecutor  # noqa: F401
