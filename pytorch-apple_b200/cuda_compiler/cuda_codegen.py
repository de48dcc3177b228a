"""Elementwise-chain encoding.

The reference generates one CUDA C kernel per chain from an expression table and
compiles it with NVRTC (cuda_compiler/cuda_codegen.py:15-142).  Here a chain is
encoded as a short program for the library's chain interpreter
(``b200_ew_chain``); nothing is compiled at run time.  ``is_fusible_elementwise``
and ``generate_fused_kernel`` keep the reference's names; the latter returns the
human-readable description that is stored in ``FusedKernelStep.source_code``.
"""

from __future__ import annotations

# opcode values of enum b200_ew_opcode (include/b200nn.h)
EW_OPCODES = {name: i + 1 for i, name in enumerate((
    "RELU", "SILU", "NEG", "RSQRT", "COS", "SIN", "ADD", "MUL", "DIV", "SUB",
    "ADD_S", "MUL_S", "DIV_S", "POW_S", "SUB_S", "CAST",
    "SIGMOID", "EXP", "SQRT", "TANH", "GELU", "RSUB_S", "MAX", "MIN"))}

_FUSIBLE = {
    "aten.relu.default", "aten.relu_.default", "aten.silu.default", "aten.silu_.default", "aten.neg.default",
    "aten.rsqrt.default", "aten.cos.default", "aten.sin.default", "aten.add.Tensor", "aten.add_.Tensor",
    "aten.mul.Tensor", "aten.mul_.Tensor", "aten.div.Tensor", "aten.sub.Tensor", "aten.pow.Tensor_Scalar",
    "aten.sigmoid.default", "aten.exp.default", "aten.sqrt.default", "aten.tanh.default", "aten.gelu.default",
}

_EXPR = {
    "relu": "max({a}, 0)", "silu": "{a} / (1 + exp(-{a}))", "neg": "-{a}", "rsqrt": "rsqrt({a})", "cos": "cos({a})",
    "sin": "sin({a})", "add": "{a} + {b}", "mul": "{a} * {b}", "div": "{a} / {b}", "sub": "{a} - {b}", "pow": "pow({a}, {b})",
    "sigmoid": "1 / (1 + exp(-{a}))", "exp": "exp({a})", "sqrt": "sqrt({a})", "tanh": "tanh({a})", "gelu": "gelu({a})",
    "to": "cast({a})", "_to_copy": "cast({a})",
}


def is_fusible_elementwise(op_type: str) -> bool:
    return op_type in _FUSIBLE


def describe_chain(nodes) -> str:
    """One line per op, e.g. ``t1 = silu(gate); y = t1 * up``."""
    lines = []
    for n in nodes:
        base = n.op_type.split(".")[1].rstrip("_") if "." in n.op_type else n.op_type
        a = n.inputs[0].name if n.inputs else "?"
        if len(n.inputs) > 1:
            b = n.inputs[1].name
        else:
            b = n.attrs.get("other", n.attrs.get("exponent", ""))
        expr = _EXPR.get(base, base + "({a})").format(a=a, b=b)
        lines.append(f"{n.outputs[0].name} = {expr}")
    return "; ".join(lines)


def generate_fused_kernel(kernel_name: str, nodes, input_names, output_name) -> str:
    """Description of the fused chain (reference signature; no source is generated)."""
    return f"{kernel_name}({', '.join(input_names)}) -> {output_name}: " + describe_chain(nodes)
