"""Weights from a safetensors checkpoint directory, as the DAG executor wants them.

Does what the reference's loaders do (examples/run_qwen_graph.py:25-82,
examples/hf_utils.py:18-140) without the hub client or the safetensors package:

* every ``*.safetensors`` file of the directory is read (all shards of
  ``model.safetensors.index.json`` when there is one) - the container format is parsed
  here: 8-byte little-endian header length, JSON header ``{name: {dtype, shape,
  data_offsets}}``, raw little-endian data; tensors are zero-copy views of a memory map;
* bfloat16 stays bfloat16: the 16-bit patterns are viewed as ``ml_dtypes.bfloat16``
  (numpy has no native bfloat16), other floats are converted to the compute dtype;
* IR weight names carry the export wrapper's ``model.`` prefix; a key that is missing is
  looked up again without that prefix;
* a tied ``lm_head.weight`` falls back to ``embed_tokens.weight``;
* ``inv_freq`` is not stored in checkpoints and is synthesised, empty ``lifted_tensor``
  placeholders (shape ``[0]``) become empty arrays.

One deliberate difference: the reference synthesises ``inv_freq`` with base 10000 whatever
the model (run_qwen_graph.py:75-77) and narrows it to bfloat16; here the base is the
checkpoint's ``rope_theta`` from ``config.json`` (10000 when absent) and the values stay
float32, because the graphs compute the rotation angle in float32.
"""

from __future__ import annotations

import json
import mmap
import os
import struct
from pathlib import Path

import numpy as np

_ST_DTYPES = {"F64": np.float64, "F32": np.float32, "F16": np.float16, "BF16": np.uint16, "I64": np.int64, "I32": np.int32,
              "I16": np.int16, "I8": np.int8, "U8": np.uint8, "BOOL": np.bool_}


def _bf16():
    import ml_dtypes

    return np.dtype(ml_dtypes.bfloat16)


def read_safetensors(path: str | os.PathLike) -> dict[str, np.ndarray]:
    """All tensors of one file; arrays are read-only views of a memory map (bf16 as ``ml_dtypes.bfloat16``)."""
    path = Path(path)
    with open(path, "rb") as f:
        head = f.read(8)
        if len(head) != 8:
            raise ValueError(f"{path}: not a safetensors file (too short)")
        (n,) = struct.unpack("<Q", head)
        size = path.stat().st_size
        if n > size - 8:
            raise ValueError(f"{path}: header length {n} exceeds the file size")
        header = json.loads(f.read(n).decode("utf-8"))
        mm = mmap.mmap(f.fileno(), 0, access=mmap.ACCESS_READ) if size > 8 + n else None
    base = 8 + n
    out: dict[str, np.ndarray] = {}
    for name, info in header.items():
        if name == "__metadata__":
            continue
        dt = _ST_DTYPES.get(info["dtype"])
        if dt is None:
            raise ValueError(f"{path}: tensor '{name}' has unsupported dtype {info['dtype']}")
        lo, hi = info["data_offsets"]
        shape = tuple(info["shape"])
        count = int(np.prod(shape)) if shape else 1
        if hi - lo != count * np.dtype(dt).itemsize or base + hi > size:
            raise ValueError(f"{path}: tensor '{name}' has inconsistent offsets")
        arr = np.frombuffer(mm, dtype=dt, count=count, offset=base + lo).reshape(shape) if count else np.zeros(shape, dt)
        out[name] = arr.view(_bf16()) if info["dtype"] == "BF16" else arr
    return out


def write_safetensors(path: str | os.PathLike, tensors: dict[str, np.ndarray], metadata: dict[str, str] | None = None) -> None:
    """Write a file in the same container format (used to build checkpoints for tests and for
    saving a seeded state dict)."""
    names = {np.dtype(v): k for k, v in _ST_DTYPES.items() if k != "BF16"}
    header: dict[str, dict] = {}
    if metadata:
        header["__metadata__"] = dict(metadata)
    blobs, at = [], 0
    for name, arr in tensors.items():
        arr = np.ascontiguousarray(arr)
        code = "BF16" if arr.dtype.name == "bfloat16" else names.get(arr.dtype)
        if code is None:
            raise TypeError(f"tensor '{name}': dtype {arr.dtype} cannot be stored")
        raw = arr.view(np.uint16).tobytes() if code == "BF16" else arr.tobytes()
        header[name] = {"dtype": code, "shape": list(arr.shape), "data_offsets": [at, at + len(raw)]}
        blobs.append(raw)
        at += len(raw)
    text = json.dumps(header, separators=(",", ":")).encode("utf-8")
    text += b" " * (-len(text) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(text)))
        f.write(text)
        for raw in blobs:
            f.write(raw)


def read_checkpoint_dir(model_dir: str | os.PathLike, wanted: set[str] | None = None) -> dict[str, np.ndarray]:
    """Tensors of a checkpoint directory.  With a shard index only the shards that hold a wanted
    key (with or without the ``model.`` prefix) are opened."""
    model_dir = Path(model_dir)
    index = model_dir / "model.safetensors.index.json"
    if index.exists():
        weight_map = json.loads(index.read_text()).get("weight_map", {})
        if wanted is None:
            files = sorted(set(weight_map.values()))
        else:
            look = set(wanted) | {k[len("model."):] for k in wanted if k.startswith("model.")}
            files = sorted({f for k, f in weight_map.items() if k in look})
    else:
        files = sorted(p.name for p in model_dir.glob("*.safetensors"))
    if not files:
        raise FileNotFoundError(f"no safetensors files under {model_dir}")
    out: dict[str, np.ndarray] = {}
    for name in files:
        out.update(read_safetensors(model_dir / name))
    return out


def load_numpy_weights(model_dir: str | os.PathLike, ir_dict: dict, compute_dtype: str = "bfloat16",
                       rope_theta: float | None = None) -> dict[str, np.ndarray]:
    """``{IR weight name: array}`` for ``DAGExecutor.load_weights`` (same contract as the
    reference's ``load_numpy_weights``, run_qwen_graph.py:25-82)."""
    model_dir = Path(model_dir)
    needed = [w for w in ir_dict.get("weights", [])]
    names = {w["name"] for w in needed}
    raw = read_checkpoint_dir(model_dir, names)
    target = _bf16() if compute_dtype == "bfloat16" else np.dtype(np.float16 if compute_dtype == "float16" else np.float32)

    def as_compute(a: np.ndarray) -> np.ndarray:
        if a.dtype.kind in "iub" or a.dtype == target:
            return a
        return a.astype(np.float32).astype(target)

    out: dict[str, np.ndarray] = {}
    for key in names:
        if key in raw:
            out[key] = as_compute(raw[key])
        elif key.startswith("model.") and key[len("model."):] in raw:
            out[key] = as_compute(raw[key[len("model."):]])
    for key in names:
        if key not in out and "lm_head.weight" in key:
            tied = key.replace("lm_head.weight", "model.embed_tokens.weight")
            if tied in out:
                out[key] = out[tied]
            elif tied.startswith("model.") and tied[len("model."):] in raw:
                out[key] = as_compute(raw[tied[len("model."):]])
    if rope_theta is None:
        cfg = model_dir / "config.json"
        rope_theta = float(json.loads(cfg.read_text()).get("rope_theta", 10000.0)) if cfg.exists() else 10000.0
    for w in needed:
        if w["name"] in out:
            continue
        if "inv_freq" in w["name"]:
            half = int(w["shape"][0])
            out[w["name"]] = (1.0 / (rope_theta ** (np.arange(half, dtype=np.float32) / half))).astype(np.float32)
        elif "lifted_tensor" in w["name"] and list(w["shape"]) == [0]:
            out[w["name"]] = np.zeros((0,), dtype=target)
    return out
