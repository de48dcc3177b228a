"""CUDA subgraph compiler for B200: IR dict -> ``CUDAProgram``.

Entry points keep the reference's names and signatures
(cuda_compiler/__init__.py:20-80): ``compile_subgraph(ir_dict, compute_dtype)``
is what ``DAGExecutor`` receives as ``compile_fn``.  The pipeline is
analyze (pattern fusion + lowering to library calls) -> plan the arena -> package.
Nothing here needs a GPU or the native library.
"""

from __future__ import annotations

from cuda_compiler.buffer_planner import plan_buffers
from cuda_compiler.cuda_program import CUDAKernelSource, CUDAProgram
from cuda_compiler.op_support import get_cuda_supported_ops as get_cuda_supported_ops
from cuda_compiler.op_support import is_cuda_op_supported as is_cuda_op_supported
from cuda_compiler.subgraph_analyzer import analyze
from npu_compiler.ir_reader import IRGraph, load_ir_from_dict


def compile_subgraph(ir_dict: dict, compute_dtype: str = "float16", donate_inputs: bool = True, fuse: bool = True,
                     keep_inputs=()) -> CUDAProgram:
    """Compile an IR dict.  ``compute_dtype`` applies to float32 graphs; a graph whose
    weights or inputs are already float16/bfloat16 computes in that type.

    ``donate_inputs``: an ``index_copy`` into a graph input that nothing else in this graph
    reads is done in place, in the caller's buffer (the KV cache of a decode step), instead of
    into a fresh copy as the reference does (cuda_templates.py:134-162).  ``keep_inputs`` names
    graph inputs that must keep their contents all the same - tensors that another partition
    of the same plan, or the caller, reads after this program ran."""
    return compile_graph(load_ir_from_dict(ir_dict), compute_dtype=compute_dtype, donate_inputs=donate_inputs, fuse=fuse,
                         keep_inputs=keep_inputs)


def compile_graph(graph: IRGraph, compute_dtype: str = "float16", donate_inputs: bool = True, fuse: bool = True,
                  keep_inputs=()) -> CUDAProgram:
    an = analyze(graph, compute_dtype, donate=donate_inputs, fuse=fuse, keep_inputs=keep_inputs)
    input_specs, output_specs, weight_specs = list(graph.graph_inputs), list(graph.graph_outputs), list(graph.weights)
    allocations = plan_buffers(an.steps, input_specs, output_specs, weight_specs, an.compute_dtype, analysis=an)
    sources, seen = [], set()
    for step in an.steps:
        name = getattr(step, "kernel_name", None)
        if name and name not in seen:
            seen.add(name)
            sources.append(CUDAKernelSource(kernel_name=name, source_code=getattr(step, "source_code", "")))
    return CUDAProgram(
        steps=an.steps,
        buffer_allocations=allocations,
        input_specs=input_specs,
        output_specs=output_specs,
        weight_specs=weight_specs,
        weight_name_mapping=dict(graph.weight_name_mapping),
        kernel_sources=sources,
        compute_dtype=an.compute_dtype,
        views=an.views,
        arena_bytes=an.arena_bytes,
        weight_preps=an.weight_preps,
        donated_inputs=an.donated,
        constants=dict(graph.constants),
    )
