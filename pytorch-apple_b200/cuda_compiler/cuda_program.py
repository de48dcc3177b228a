"""Program model handed from the compiler to the executor.

The step classes and ``CUDAProgram`` keep the names and fields of the reference
model (cuda_compiler/cuda_program.py:15-111) so that code written against it - the
DAG executor, the tests - keeps working.  What differs is what a step *means*:
there is no CUDA source to JIT.  ``kernel_name`` names an entry point family of the
native library, ``source_code`` holds a one-line human-readable description of the
fused computation (it is never compiled), and ``params`` carries everything the
executor needs to bind the call: operand tensor names resolve through
``CUDAProgram.views`` to (buffer, offset, shape, strides, dtype).
"""

from __future__ import annotations

import dataclasses
import json
from dataclasses import dataclass, field
from pathlib import Path

from npu_compiler.ir_reader import TensorSpec


@dataclass
class TensorView:
    """Where a tensor lives: ``buffer`` is an arena allocation, a graph input or a
    weight placeholder; offset and strides are in elements of ``dtype``."""

    buffer: str
    offset: int
    shape: tuple[int, ...]
    strides: tuple[int, ...]
    dtype: str

    @property
    def numel(self) -> int:
        n = 1
        for s in self.shape:
            n *= s
        return n

    def is_contiguous(self) -> bool:
        expect = 1
        for extent, stride in zip(reversed(self.shape), reversed(self.strides)):
            if extent != 1 and stride != expect:
                return False
            expect *= extent
        return True


@dataclass
class BufferAllocation:
    name: str
    shape: list[int]
    dtype: str = "float16"
    size_bytes: int = 0
    offset: int = -1            # byte offset in the per-GPU arena (-1: not arena backed)
    first_step: int = 0         # liveness interval in step indices, used by the planner
    last_step: int = 0
    persistent: bool = False    # never shares memory; zero-filled once (padding, scratch)


@dataclass
class CUDAKernelSource:
    kernel_name: str
    source_code: str


@dataclass
class CUBLASStep:
    blas_type: str  # "gemm", "gemm_batched", "conv2d", "attention"
    input_buffer_names: list[str]
    output_buffer_name: str
    params: dict


@dataclass
class FusedKernelStep:
    kernel_name: str
    source_code: str
    input_buffer_names: list[str]
    output_buffer_name: str
    total_elements: int
    block_size: int = 256
    params: dict = field(default_factory=dict)


@dataclass
class ReductionKernelStep:
    kernel_name: str
    source_code: str
    input_buffer_names: list[str]
    output_buffer_name: str
    params: dict
    block_size: int = 256


@dataclass
class AliasStep:
    input_buffer_name: str
    output_buffer_name: str
    input_shape: list[int]
    output_shape: list[int]


@dataclass
class SpecialKernelStep:
    kernel_name: str
    source_code: str
    input_buffer_names: list[str]
    output_buffer_name: str
    output_buffer_names: list[str] = field(default_factory=list)
    params: dict = field(default_factory=dict)
    block_size: int = 256
    grid_dim: tuple[int, ...] = (1,)


ExecStep = CUBLASStep | FusedKernelStep | ReductionKernelStep | AliasStep | SpecialKernelStep


@dataclass
class WeightPrep:
    """One-off transformation of uploaded weights, run when a weight set is first seen."""

    kind: str                 # "conv_fold" | "concat_rows"
    inputs: list[str | None]  # weight placeholder names (None = absent operand)
    outputs: list[str]        # names of executor-owned buffers it fills
    params: dict = field(default_factory=dict)


@dataclass
class CUDAProgram:
    steps: list[ExecStep]
    buffer_allocations: list[BufferAllocation]
    input_specs: list[TensorSpec]
    output_specs: list[TensorSpec]
    weight_specs: list[TensorSpec]
    weight_name_mapping: dict[str, str]
    kernel_sources: list[CUDAKernelSource] = field(default_factory=list)
    compute_dtype: str = "float16"
    # --- additions -------------------------------------------------------------
    views: dict[str, TensorView] = field(default_factory=dict)
    arena_bytes: int = 0
    weight_preps: list[WeightPrep] = field(default_factory=list)
    donated_inputs: dict[str, str] = field(default_factory=dict)  # output name -> graph input it overwrites
    constants: dict = field(default_factory=dict)

    @property
    def kernel_calls(self):
        """Reference-compatible alias for ``steps``."""
        return self.steps

    # -- serialisation ------------------------------------------------------------------
    # The reference can store a compiled Metal program (``CompiledProgram.save / load``,
    # npu_compiler/compiled_program.py:49-117: a JSON file tagged with format and version); its
    # CUDA program has no such pair.  Same idea here: everything the executor needs - steps with
    # their resolved views, the arena plan, weight preparations - as one JSON document, so that a
    # serving process can skip export, pattern matching and planning.
    FORMAT, VERSION = "b200prog", 1

    def to_dict(self) -> dict:
        return {"format": self.FORMAT, "version": self.VERSION, "program": _encode(self)}

    def save(self, path: str) -> None:
        Path(path).write_text(json.dumps(self.to_dict()))

    @classmethod
    def from_dict(cls, data: dict) -> "CUDAProgram":
        if data.get("format") != cls.FORMAT:
            raise ValueError(f"not a {cls.FORMAT} document (format = {data.get('format')!r})")
        if data.get("version") != cls.VERSION:
            raise ValueError(f"{cls.FORMAT} version {data.get('version')} is not supported (this build reads version {cls.VERSION})")
        prog = _decode(data["program"])
        if not isinstance(prog, cls):
            raise ValueError("document does not hold a CUDAProgram")
        return prog

    @classmethod
    def load(cls, path: str) -> "CUDAProgram":
        return cls.from_dict(json.loads(Path(path).read_text()))


_SERIALISABLE = {c.__name__: c for c in (TensorView, BufferAllocation, CUDAKernelSource, CUBLASStep, FusedKernelStep, ReductionKernelStep,
                                         AliasStep, SpecialKernelStep, WeightPrep, CUDAProgram, TensorSpec)}


def _encode(obj):
    """JSON form of a program tree: dataclasses and tuples are tagged so that ``_decode`` restores them exactly."""
    if dataclasses.is_dataclass(obj) and not isinstance(obj, type):
        name = type(obj).__name__
        if name not in _SERIALISABLE:
            raise TypeError(f"cannot serialise {name}")
        return {"__dc__": name, **{f.name: _encode(getattr(obj, f.name)) for f in dataclasses.fields(obj)}}
    if isinstance(obj, tuple):
        return {"__tuple__": [_encode(v) for v in obj]}
    if isinstance(obj, list):
        return [_encode(v) for v in obj]
    if isinstance(obj, dict):
        if not all(isinstance(k, str) for k in obj):
            raise TypeError("only string keys can be serialised")
        return {k: _encode(v) for k, v in obj.items()}
    if isinstance(obj, (set, frozenset)):
        return {"__set__": sorted(_encode(v) for v in obj)}
    if obj is None or isinstance(obj, (bool, int, float, str)):
        return obj
    raise TypeError(f"cannot serialise a value of type {type(obj).__name__}")


def _decode(obj):
    if isinstance(obj, list):
        return [_decode(v) for v in obj]
    if isinstance(obj, dict):
        if "__tuple__" in obj:
            return tuple(_decode(v) for v in obj["__tuple__"])
        if "__set__" in obj:
            return set(_decode(v) for v in obj["__set__"])
        if "__dc__" in obj:
            cls = _SERIALISABLE[obj["__dc__"]]
            return cls(**{k: _decode(v) for k, v in obj.items() if k != "__dc__"})
        return {k: _decode(v) for k, v in obj.items()}
    return obj
