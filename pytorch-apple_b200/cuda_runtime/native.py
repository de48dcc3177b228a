"""ctypes binding of ``libb200nn.so`` (declared in include/b200nn.h).

The library is the only compute path: if it cannot be loaded the runtime raises,
there is no fallback.  ``load()`` declares argument types for every entry point so
that a wrong call fails in Python rather than in the kernel.
"""

from __future__ import annotations

import ctypes as C
import os
from pathlib import Path

LIB_NAME = "libb200nn.so"
MAX_DIMS = 6
EW_MAX_INPUTS = 4
EW_MAX_OPS = 12

DTYPE_CODES = {"float32": 0, "float16": 1, "bfloat16": 2, "int32": 3, "int64": 4, "uint8": 5, "bool": 5}
DTYPE_BYTES = {"float32": 4, "float16": 2, "bfloat16": 2, "int32": 4, "int64": 8, "uint8": 1, "bool": 1}

EPI_RELU = 1
EPI_SILU_MUL = 2
EPI_GLU = 4
EPI_W_STATIC = 8


class Tensor(C.Structure):
    """``b200_tensor``."""

    _fields_ = [("data", C.c_void_p), ("dtype", C.c_int32), ("ndim", C.c_int32),
                ("shape", C.c_int64 * MAX_DIMS), ("stride", C.c_int64 * MAX_DIMS)]


class EwOp(C.Structure):
    """``b200_ew_op``."""

    _fields_ = [("opcode", C.c_int32), ("a", C.c_int32), ("b", C.c_int32), ("round_dtype", C.c_int32), ("imm", C.c_float)]


_vp, _i, _i64, _f = C.c_void_p, C.c_int, C.c_int64, C.c_float
_TP = C.POINTER(Tensor)
_I64P = C.POINTER(C.c_int64)

# name -> (restype, argtypes); every symbol include/b200nn.h declares
SIGNATURES = {
    "b200_version": (_i, []),
    "b200_last_error": (C.c_char_p, []),
    "b200_device_info": (_i, [_i, C.POINTER(_i), C.POINTER(_i), C.POINTER(_i), C.POINTER(_i64)]),
    "b200_debug_device_error": (_i, [C.POINTER(_i), _i]),
    "b200_debug_wait_timeout": (_i, [_i, _vp]),
    "b200_ew_chain": (_i, [_TP, _TP, _i, C.POINTER(EwOp), _i, _vp]),
    "b200_strided_copy": (_i, [_TP, _TP, _vp]),
    "b200_fill": (_i, [_vp, _i64, C.c_double, _i, _vp]),
    "b200_rmsnorm": (_i, [_vp, _vp, _vp, _i64, _i64, _i64, _i64, _f, _i, _i, _vp]),
    "b200_softmax": (_i, [_vp, _vp, _vp, _i64, _i64, _i64, _i64, _i64, _i64, _i64, _f, _i, _i, _i, _i, _vp]),
    "b200_mean_last_dim": (_i, [_vp, _vp, _i64, _i64, _i, _i, _vp]),
    "b200_embedding": (_i, [_vp, _vp, _vp, _i64, _i64, _i64, _i, _vp]),
    "b200_index_copy": (_i, [_vp, _vp, _vp, _vp, _i64, _i64, _i64, _i64, _i64, _i64, _i, _i, _vp]),
    "b200_argmax_rows": (_i, [_vp, _vp, _i64, _i64, _i64, _i, _vp]),
    "b200_rope_table": (_i, [_vp, _vp, _vp, _vp, _i64, _i, _i, _i, _vp]),
    "b200_rope_rotate": (_i, [_TP, _vp, _vp, _vp, _vp, _vp, _i64, _i, _vp]),
    "b200_rope_rotate_pair": (_i, [_TP, _TP, _vp, _vp, _vp, _vp, _vp]),
    "b200_qkv_rope_cache": (_i, [_TP, _TP, _TP, _vp, _vp, _vp, _vp, _vp, _vp, _i64, _i, _vp]),
    "b200_max_pool2d": (_i, [_TP, _TP, _i, _i, _i, _i, _i, _i, _vp]),
    "b200_adaptive_avg_pool2d": (_i, [_TP, _TP, _vp]),
    "b200_batch_norm": (_i, [_TP, _TP, _vp, _vp, _vp, _vp, _f, _i, _i, _vp]),
    "b200_conv_weight_prep": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _f, _i, _i, _i, _vp]),
    "b200_linear": (_i, [_vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _i64, _i64, _i64, _i64, _i, _i, _i, _vp, _i64, _vp, _i64, _vp]),
    "b200_linear_workspace_bytes": (_i64, [_i64, _i64, _i64]),
    "b200_linear_rmsnorm": (_i, [_vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _i64, _i64, _i64, _i64, _i, _i, _i, _vp, _i64, _vp, _vp, _i64, _f, _i, _vp]),
    "b200_linear_norm": (_i, [_vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _i64, _i64, _i64, _i64, _i, _i, _i, _f, _vp, _i, _vp, _vp]),
    "b200_linear_qkv_rope": (_i, [_vp, _vp, _vp, _i64, _i64, _i64, _i64, _i64, _i, _i, _i, _f, _vp, _i, _vp, _vp, _vp, _vp, _vp, _vp, _i64, _i, _i, _i,
                                  _vp]),
    "b200_matmul_strided": (_i, [_vp, _vp, _vp, _i64, _i64, _i64, _i64, _i64, _I64P, _I64P, _I64P, _i, _vp]),
    "b200_conv2d_nhwc": (_i, [_vp, _vp, _vp, _vp, _vp] + [_i] * 16 + [_vp]),
    "b200_attn_decode": (_i, [_vp, _vp, _vp, _vp, _vp, _i64, _i, _i, _i64, _i, _i64, _i64, _i64, _i64, _f, _i, _vp, _i64, _vp]),
    "b200_attn_decode_noalloc": (_i, [_vp, _vp, _vp, _vp, _vp, _i64, _i, _i, _i64, _i, _i64, _i64, _i64, _i64, _f, _i, _vp]),
    "b200_attn_decode_workspace_bytes": (_i64, [_i64, _i, _i, _i64, _i]),
    "b200_attn_prefill": (_i, [_vp, _vp, _vp, _vp, _vp, _i64, _i, _i, _i64, _i64, _i, _I64P, _I64P, _I64P, _i64, _i64, _f, _i, _vp]),
}

_lib = None
_test_override = None  # (library object, torch device string) installed by the test-suite


def library_path() -> Path:
    env = os.environ.get("B200NN_LIBRARY")
    return Path(env) if env else Path(__file__).resolve().parent / LIB_NAME


def load():
    """The loaded library with typed entry points.  Raises ``RuntimeError`` when the
    shared object is missing or does not export a declared symbol."""
    global _lib
    if _test_override is not None:
        return _test_override[0]
    if _lib is not None:
        return _lib
    path = library_path()
    if not path.exists():
        raise RuntimeError(f"{path} not found: build it with `python build_native.py` (needs nvcc); "
                           "there is no fallback path without the native kernel library")
    try:
        lib = C.CDLL(str(path))
    except OSError as exc:
        raise RuntimeError(f"cannot load {path}: {exc}") from exc
    for name, (restype, argtypes) in SIGNATURES.items():
        try:
            fn = getattr(lib, name)
        except AttributeError as exc:
            raise RuntimeError(f"{path} does not export {name}") from exc
        fn.restype = restype
        fn.argtypes = argtypes
    _lib = lib
    return lib


def device_string(device_id: int = 0) -> str:
    if _test_override is not None:
        return _test_override[1]
    return f"cuda:{device_id}"


def install_test_library(lib, device: str = "cpu") -> None:
    """Test seam: route calls to a stand-in object (used by the CPU test-suite to
    exercise the host logic without a GPU).  Never used by the product."""
    global _test_override
    _test_override = None if lib is None else (lib, device)


def check(rc: int, what: str = "") -> None:
    if rc != 0:
        msg = load().b200_last_error()
        msg = msg.decode() if isinstance(msg, bytes) else str(msg)
        raise RuntimeError(f"b200nn call failed ({rc}) {what}: {msg}")


def make_tensor(ptr: int, dtype: str, shape, strides) -> Tensor:
    if len(shape) > MAX_DIMS:
        raise ValueError(f"tensor rank {len(shape)} exceeds {MAX_DIMS}")
    t = Tensor()
    t.data = ptr
    t.dtype = DTYPE_CODES[dtype]
    t.ndim = len(shape)
    for i, (s, st) in enumerate(zip(shape, strides)):
        t.shape[i] = int(s)
        t.stride[i] = int(st)
    return t
