"""IR graph -> ordered list of library-call steps.

Same role and entry point as the reference analyzer
(cuda_compiler/subgraph_analyzer.py:797-981, ``analyze_subgraph(graph) -> steps``):
pattern pre-passes, greedy fusion of single-consumer elementwise chains, one step
builder per op category.  The output differs in kind: every step names an entry
point of the fixed native kernel library and carries resolved tensor views, instead
of CUDA source text for NVRTC.

Lowering rules that have no counterpart in the reference:

* view-like ops (reshape, transpose, slice, expand, unsqueeze, getitem, ...) become
  stride arithmetic at compile time; a copy kernel is emitted only when the result
  cannot be expressed as strides;
* activations of convolution networks are stored channels-last (NHWC) - an NCHW
  shaped view with permuted strides - and inference batch-norm is folded into the
  convolution weights by a one-off weight-preparation step;
* ``index_copy`` into a graph input that nothing else reads is done in place (the
  updated cache that the graph returns *is* the input buffer).
"""

from __future__ import annotations

import math
from dataclasses import dataclass, field

from cuda_compiler import views as V
from cuda_compiler.cuda_codegen import EW_OPCODES, describe_chain, is_fusible_elementwise
from cuda_compiler.cuda_program import (
    AliasStep,
    BufferAllocation,
    CUBLASStep,
    FusedKernelStep,
    ReductionKernelStep,
    SpecialKernelStep,
    TensorView,
    WeightPrep,
)
from cuda_compiler.op_classify import OpCategory, classify_op
from cuda_compiler.patterns import (
    ADD_OPS,
    DEFAULT_FAMILIES,
    NOOP_OPS,
    PASSTHROUGH_OPS,
    GraphIndex,
    apply_patterns,
    fuse_qkv_post,
    fuse_rope_pair,
    group_linears,
)
from npu_compiler.ir_reader import IRGraph, OpNode, TensorSpec

FLOAT_DTYPES = ("float32", "float16", "bfloat16")
DTYPE_BYTES = {"float32": 4, "float16": 2, "bfloat16": 2, "int32": 4, "int64": 8, "bool": 1, "uint8": 1}
MAX_CHAIN_OPS = 12
MAX_CHAIN_INPUTS = 4


def infer_compute_dtype(graph: IRGraph, requested: str | None) -> str:
    """A graph whose weights/inputs are already half precision computes in that type;
    a float32 graph computes in ``requested`` (default float16, as the reference does
    for every graph - cuda_compiler/__init__.py:20)."""
    for spec in list(graph.weights) + list(graph.graph_inputs):
        if spec.dtype in ("bfloat16", "float16"):
            return spec.dtype
    return requested or "float16"


@dataclass
class Analysis:
    steps: list = field(default_factory=list)
    views: dict[str, TensorView] = field(default_factory=dict)
    buffers: dict[str, BufferAllocation] = field(default_factory=dict)
    weight_preps: list[WeightPrep] = field(default_factory=list)
    donated: dict[str, str] = field(default_factory=dict)
    compute_dtype: str = "float16"
    arena_bytes: int = 0
    step_tensors: list[list[str]] = field(default_factory=list)  # tensor names each step touches


class _Lowering:
    def __init__(self, graph: IRGraph, compute_dtype: str, donate: bool = True, fuse: bool = True, keep_inputs=()):
        self.graph = graph
        self.cd = compute_dtype
        self.donate = donate
        self.keep_inputs = frozenset(keep_inputs)   # graph inputs somebody outside this graph still reads
        self.fuse = fuse
        self.out = Analysis(compute_dtype=compute_dtype)
        low_precision = any(s.dtype in ("bfloat16", "float16") for s in list(graph.weights) + list(graph.graph_inputs))
        self.narrow_f32 = (not low_precision) and compute_dtype in ("float16", "bfloat16")
        self.external: set[str] = set()
        self._n_scratch = 0
        # graph inputs and weights are their own buffers
        for spec in graph.graph_inputs:
            self._external_view(spec.name, spec)
        key_spec = {w.name: w for w in graph.weights}
        placeholders = {key: ph for ph, key in graph.weight_name_mapping.items()}
        for w in graph.weights:
            self._external_view(placeholders.get(w.name, w.name), w, weight=True)
        for ph, key in graph.weight_name_mapping.items():
            if ph not in self.out.views and key in key_spec:
                self._external_view(ph, key_spec[key], weight=True)
        self.weight_names = {n for n in self.out.views if n not in {s.name for s in graph.graph_inputs}}

    # -- dtype / buffers -------------------------------------------------------
    def sd(self, ir_dtype: str) -> str:
        """Storage dtype of an IR dtype."""
        if ir_dtype == "bool":
            return "uint8"
        if ir_dtype == "float32" and self.narrow_f32:
            return self.cd
        if ir_dtype == "float64":
            return "float32"
        return ir_dtype

    def _external_view(self, name: str, spec: TensorSpec, weight: bool = False) -> None:
        shape = tuple(int(s) for s in spec.shape)
        self.out.views[name] = TensorView(name, 0, shape, V.contiguous_strides(shape), self.sd(spec.dtype))
        self.external.add(name)

    def alloc(self, name: str, shape, dtype: str, strides=None, persistent: bool = False) -> TensorView:
        shape = tuple(int(s) for s in shape)
        strides = tuple(strides) if strides is not None else V.contiguous_strides(shape)
        nbytes = max(1, math.prod(shape)) * DTYPE_BYTES[dtype]
        self.out.buffers[name] = BufferAllocation(name=name, shape=list(shape), dtype=dtype, size_bytes=nbytes,
                                                  persistent=persistent)
        view = TensorView(name, 0, shape, strides, dtype)
        self.out.views[name] = view
        return view

    def scratch(self, nbytes: int, tag: str, persistent: bool = False) -> str:
        self._n_scratch += 1
        name = f"__scratch_{tag}_{self._n_scratch}"
        self.alloc(name, (int(nbytes),), "uint8", persistent=persistent)
        return name

    def view(self, name: str) -> TensorView:
        return self.out.views[name]

    def emit(self, step, tensors: list[str]) -> None:
        self.out.steps.append(step)
        self.out.step_tensors.append([t for t in tensors if t is not None])

    def alias(self, node: OpNode, src: str, view: TensorView) -> None:
        out = node.outputs[0]
        self.out.views[out.name] = view
        self.emit(AliasStep(src, out.name, list(self.view(src).shape), list(view.shape)), [src, out.name])

    # -- helpers -----------------------------------------------------------------
    def contiguous(self, name: str, tag: str = "contig") -> str:
        """Name of a contiguous tensor holding ``name`` (copying if needed)."""
        v = self.view(name)
        if v.is_contiguous():
            return name
        self._n_scratch += 1
        new = f"{name}__{tag}{self._n_scratch}"
        self.alloc(new, v.shape, v.dtype)
        self.copy(name, new)
        return new

    def copy(self, src: str, dst: str) -> None:
        self.emit(SpecialKernelStep("strided_copy", "out[idx] = in[idx]", [src], dst,
                                    params={"op": "strided_copy", "in_view": self.view(src), "out_view": self.view(dst)}),
                  [src, dst])

    def as_2d(self, name: str) -> tuple[str, TensorView]:
        """[..., K] -> [M, K] with unit inner stride, copying only if unavoidable."""
        v = self.view(name)
        K = v.shape[-1] if v.shape else 1
        M = v.numel // max(K, 1)
        r = V.try_reshape(v, (M, K))
        if r is None or (r.strides[1] != 1 and K > 1):
            name = self.contiguous(name)
            r = V.try_reshape(self.view(name), (M, K))
        return name, r

    def out_like(self, node_out: TensorSpec, like: str | None = None) -> TensorView:
        dtype = self.sd(node_out.dtype)
        strides = None
        if like is not None:
            strides = V.like_strides(tuple(node_out.shape), self.view(like))
        return self.alloc(node_out.name, node_out.shape, dtype, strides)

    # -- driver ------------------------------------------------------------------
    def run(self) -> Analysis:
        nodes = [n for n in self.graph.nodes if n.op_type not in NOOP_OPS]
        if self.fuse:
            nodes = apply_patterns(nodes, self.graph, DEFAULT_FAMILIES)
            nodes = group_linears(nodes, self.graph)
            nodes = fuse_qkv_post(nodes, self.graph)
            nodes = fuse_rope_pair(nodes, self.graph)
        self.gi = GraphIndex.build(nodes, self.graph)
        self._chain_done: set[int] = set()
        for node in nodes:
            if id(node) in self._chain_done:
                continue
            self.lower(node)
        if self.fuse:
            self._fold_rmsnorm_into_decode_linears()
            self._fuse_rope_into_qkv_linear()
            self._append_rmsnorm_to_splitk_linears()
        return self.out

    def _fuse_rope_into_qkv_linear(self) -> None:
        """Decode shapes (one token per sequence, at most 64 sequences, head dimension 128): the merged
        q/k/v projection is followed by one small kernel that rotates q and k and writes the new K / V
        rows into the caches.  With 128-wide GEMM tiles a tile is one head, so the GEMM's final pass
        can do that itself (``b200_linear_qkv_rope``): same roundings, one launch less per layer.  The
        fused step takes the place of the rope / cache step (its table and index operands may be
        produced after the projection's position in the step list)."""
        steps, touched = self.out.steps, self.out.step_tensors
        producer: dict[str, int] = {}
        readers: dict[str, set[int]] = {}
        for i, st in enumerate(steps):
            if isinstance(st, AliasStep):
                continue
            outs = set(getattr(st, "output_buffer_names", None) or [st.output_buffer_name])
            for name in touched[i]:
                v = self.out.views.get(name)
                b = v.buffer if v is not None else name
                if name in outs:
                    producer[b] = i if b not in producer else -1
                else:
                    readers.setdefault(b, set()).add(i)
        drop: set[int] = set()
        for i, st in enumerate(steps):
            p = getattr(st, "params", None) or {}
            if p.get("op") != "qkv_post" or not p.get("in_place"):
                continue
            q, k, v = p["q"], p["k"], p["v"]
            B, Hq, T, D = q.shape
            Hkv = k.shape[1]
            N = (Hq + 2 * Hkv) * D
            if T != 1 or D != 128 or B > 64 or not (q.buffer == k.buffer == v.buffer) or v.shape[1] != Hkv:
                continue
            src = producer.get(q.buffer, -1)
            if src < 0 or src >= i or src in drop or readers.get(q.buffer, set()) != {i}:
                continue
            lp = getattr(steps[src], "params", None) or {}
            if lp.get("op") != "linear" or lp.get("glu") or lp.get("relu") or lp.get("residual") is not None or lp.get("aux") is not None \
                    or lp.get("sumsq_out") is not None or lp["M"] != B or lp["N"] != N or lp["y"].buffer != q.buffer:
                continue
            y = lp["y"]
            head_major = all(t.strides[1] == D and t.strides[3] == 1 and (B == 1 or t.strides[0] == N) for t in (q, k, v))
            if not head_major or not y.is_contiguous() or q.offset != y.offset or k.offset != y.offset + Hq * D or v.offset != y.offset + (Hq + Hkv) * D:
                continue
            # nothing between the projection and the rope step may depend on the move: the projection's output has no other reader
            params = dict(lp)
            params.update(op="linear_qkv_rope", rope={k_: p[k_] for k_ in ("cos", "sin", "q_out", "k_cache", "v_cache", "index", "cache_len")},
                          Hq=Hq, Hkv=Hkv, source="rope(q), cache writes folded in: " + lp.get("source", ""))
            names = list(dict.fromkeys(list(steps[src].input_buffer_names) + [n for n in st.input_buffer_names if self.out.views.get(n) is None
                                                                                or self.out.views[n].buffer != q.buffer]))
            steps[i] = SpecialKernelStep("gemm_tc5_kernel", "q/k/v projection -> rope(q); key cache[pos] = rope(k); value cache[pos] = v  (in place)",
                                         names, st.output_buffer_name, output_buffer_names=list(st.output_buffer_names), params=params)
            touched[i] = list(dict.fromkeys([n for n in touched[src]] + [n for n in touched[i]]))
            drop.add(src)
        if drop:
            self.out.steps = [s for i, s in enumerate(steps) if i not in drop]
            self.out.step_tensors = [t for i, t in enumerate(touched) if i not in drop]

    def _fold_rmsnorm_into_decode_linears(self) -> None:
        """Decode shapes (M <= 64): an RMSNorm between two GEMMs costs a kernel launch for a few
        hundred KB.  Where the normalised tensor feeds exactly one GEMM and its input x comes out
        of a GEMM, the producing GEMM also writes sum-of-squares partials of its output rows
        (``sumsq_out``, one fp32 per row and 64 columns); the consuming GEMM reads the
        un-normalised x, uses weights with the gain folded into their columns (weight
        preparation, once per weight set) and scales its output rows by 1/rms(x) from the
        partials, since (r x * g) W^T = r (x (W * g)^T) (``b200_linear_norm``).  The normalised
        activations are no longer rounded to the 16-bit type on the way, so results differ from
        the unfused kernels by rounding only; ``fuse=False`` keeps the unfused kernels."""
        steps = self.out.steps
        touched = self.out.step_tensors

        def buffer_of(name: str) -> str:
            v = self.out.views.get(name)
            return v.buffer if v is not None else name

        producer: dict[str, int] = {}          # buffer -> the one step that writes it (-1: several)
        readers: dict[str, list[int]] = {}     # buffer -> steps that read it
        for i, st in enumerate(steps):
            if isinstance(st, AliasStep):
                continue
            outs = set(getattr(st, "output_buffer_names", None) or [st.output_buffer_name])
            for name in touched[i]:
                b = buffer_of(name)
                if name in outs:
                    producer[b] = i if b not in producer else -1
                elif i not in readers.setdefault(b, []):
                    readers[b].append(i)
        graph_outputs = {o.name for o in self.graph.graph_outputs}
        drop: set[int] = set()
        for i, st in enumerate(steps):
            p = getattr(st, "params", None) or {}
            if p.get("op") != "rmsnorm" or not p.get("round_mid"):
                continue
            y_name = st.output_buffer_name
            x_view = p["x"]
            rows, cols = p["rows"], p["cols"]
            users = readers.get(p["y"].buffer, [])
            if y_name in graph_outputs or len(users) != 1 or producer.get(p["y"].buffer) != i or rows > 64 or cols % 64 or cols > 2048:
                continue
            cons = steps[users[0]]
            cp = getattr(cons, "params", None) or {}
            if cp.get("op") != "linear" or cp.get("aux") is not None or cp["x"].buffer != p["y"].buffer or cp["x"].offset != p["y"].offset \
                    or cp["K"] != cols or cp["M"] != rows or cp.get("norm") or x_view.strides[-1] != 1 or x_view.offset % 8 \
                    or (rows > 1 and x_view.strides[0] % 8):
                continue
            if cp["N"] >= 2 * 148 * 256:
                continue   # a vocabulary-sized projection runs on the persistent kernel, which carries no row scaling (91 against 115 us)
            # the producer of x: a GEMM writing exactly this [rows, cols] tensor, alone
            src = producer.get(x_view.buffer, -1)
            if src < 0:
                continue
            pp = getattr(steps[src], "params", None) or {}
            if pp.get("op") != "linear" or pp.get("glu") or pp.get("aux") is not None or pp["M"] != rows or pp["N"] != cols \
                    or pp["y"].offset != x_view.offset or pp["y"].buffer != x_view.buffer or pp.get("sumsq_out") is not None:
                continue
            n_part = cols // 64
            sq = self.alloc(f"{y_name}__sumsq", (rows, n_part), "float32")
            pp["sumsq_out"] = sq
            touched[src].append(sq.buffer)
            cp["norm"] = {"eps": float(p["eps"]), "sumsq": sq, "cols": n_part}
            cp["x"] = x_view
            # the gain goes into the columns of the consumer's weights
            prep = next((wp for wp in self.out.weight_preps if cp["w"] in wp.outputs), None)
            if prep is not None and prep.kind in ("concat_rows", "interleave_rows") and "col_scale" not in prep.params:
                prep.params["col_scale"] = p["w"]
            else:
                scaled = f"{cp['w']}__x_{p['w']}"
                if scaled not in self.out.views:
                    wv = self.view(cp["w"])
                    self.out.weight_preps.append(WeightPrep("scale_cols", [cp["w"], p["w"]], [scaled],
                                                            {"rows": int(wv.shape[0]), "cols": int(wv.shape[1]), "dtype": cp["y"].dtype}))
                    self.out.views[scaled] = TensorView(scaled, 0, tuple(wv.shape), V.contiguous_strides(wv.shape), cp["y"].dtype)
                cp["w"] = scaled
            names = [n for n in touched[users[0]] if n != y_name] + [x_view.buffer, sq.buffer]
            touched[users[0]] = names
            if hasattr(cons, "input_buffer_names"):
                cons.input_buffer_names = [x_view.buffer if n == y_name else n for n in cons.input_buffer_names]
            cp["source"] = "rmsnorm(x) folded in: " + cp.get("source", "")
            drop.add(i)
        if drop:
            self.out.steps = [s for i, s in enumerate(steps) if i not in drop]
            self.out.step_tensors = [t for i, t in enumerate(touched) if i not in drop]

    @staticmethod
    def _pair_splitk_shape(M: int, N: int, K: int) -> bool:
        """The shapes the library runs on 256 x 256 CTA-pair tiles with split-K and a reduce kernel (few
        tiles, long reduction: the down projection of a 512- or 1024-token prompt), and whose rows that
        kernel can normalise.  A wrong guess costs nothing but a plan that promises a fusion the library
        then runs as two kernels."""
        tiles = -(-M // 256) * -(-N // 256)
        return M > 128 and 256 <= N <= 2048 and N % 8 == 0 and K >= 4096 and 12 <= tiles < 37

    def _append_rmsnorm_to_splitk_linears(self) -> None:
        """A GEMM whose partial sums are added up by a second kernel, followed directly by the RMSNorm
        of its result (down projection + residual -> the next layer's input norm at prefill): the
        adding kernel normalises the finished row as well (``b200_linear_rmsnorm``), same roundings,
        one launch less.  The GEMM result itself is still written - the residual stream reads it."""
        steps, touched = self.out.steps, self.out.step_tensors
        drop: set[int] = set()
        last = -1   # the last step that is not an alias
        for i, st in enumerate(steps):
            if isinstance(st, AliasStep):
                continue
            prev, last = last, i
            p = getattr(st, "params", None) or {}
            if p.get("op") != "rmsnorm" or prev < 0 or prev in drop:
                continue
            lp = getattr(steps[prev], "params", None) or {}
            if lp.get("op") != "linear" or lp.get("glu") or lp.get("aux") is not None or lp.get("norm") or lp.get("sumsq_out") is not None \
                    or lp.get("norm_tail") or not isinstance(steps[prev], CUBLASStep):
                continue
            x, y, ly = p["x"], p["y"], lp["y"]
            M, N, K = lp["M"], lp["N"], lp["K"]
            if p["rows"] != M or p["cols"] != N or not self._pair_splitk_shape(M, N, K):
                continue
            row = lambda v: v.strides[-2] if len(v.shape) >= 2 and v.shape[-2] > 1 else v.shape[-1]
            if x.buffer != ly.buffer or x.offset != ly.offset or x.dtype != ly.dtype or x.strides[-1] != 1 or row(x) != row(ly) \
                    or y.strides[-1] != 1 or row(y) % 8 or y.offset % 8 or row(y) != N:
                continue
            params = dict(lp)
            params["norm_tail"] = {"w": p["w"], "y": y, "eps": float(p["eps"]), "round_mid": bool(p["round_mid"])}
            params["source"] = lp.get("source", "") + " ; rmsnorm(result) * gain"
            names = list(dict.fromkeys(list(steps[prev].input_buffer_names) + [p["w"]]))
            # one step with two results: the GEMM's own and the normalised rows
            steps[prev] = SpecialKernelStep("gemm_pair_kernel", "x @ W^T (+ b, + residual) split over CTA pairs; the kernel that adds up the "
                                            "partial sums also writes rmsnorm(result) * gain", names, steps[prev].output_buffer_name,
                                            output_buffer_names=[steps[prev].output_buffer_name, st.output_buffer_name], params=params)
            touched[prev] = list(dict.fromkeys(list(touched[prev]) + [n for n in touched[i]]))
            drop.add(i)
            last = prev
        if drop:
            self.out.steps = [s for i, s in enumerate(steps) if i not in drop]
            self.out.step_tensors = [t for i, t in enumerate(touched) if i not in drop]

    def lower(self, node: OpNode) -> None:
        op = node.op_type
        if op.startswith("b200."):
            getattr(self, "lower_" + op.split(".")[1])(node)
            return
        cat = classify_op(op)
        if cat == OpCategory.NOOP:
            return
        if cat == OpCategory.SHAPE_ALIAS:
            self.lower_alias(node)
        elif cat == OpCategory.ELEMENTWISE:
            self.lower_chain(node)
        elif cat == OpCategory.REDUCTION:
            self.lower_reduction(node)
        elif cat == OpCategory.ANCHOR_BLAS:
            self.lower_blas(node)
        else:
            self.lower_special(node)

    # -- view-like ops ---------------------------------------------------------------
    def lower_alias(self, node: OpNode) -> None:
        op, a = node.op_type, node.attrs
        out = node.outputs[0]
        if op == "<built-in function getitem>":
            idx = a.get("index", 0)
            src = node.inputs[idx if idx < len(node.inputs) else 0].name
            return self.alias(node, src, self.view(src))
        if op == "aten.cat.default":
            return self.lower_cat(node)
        src = node.inputs[0].name
        v = self.view(src)
        nd = len(v.shape)
        if op in ("aten.to.dtype", "aten._to_copy.default"):
            if self.sd(out.dtype) == v.dtype:
                return self.alias(node, src, v)
            return self.lower_chain(node)
        if op in PASSTHROUGH_OPS or op in ("aten.lift_fresh_copy.default",):
            if op in ("aten.contiguous.default", "aten.clone.default") and not v.is_contiguous():
                self.alloc(out.name, out.shape, v.dtype)
                return self.copy(src, out.name)
            return self.alias(node, src, v)
        if op in ("aten.reshape.default", "aten.view.default", "aten._unsafe_view.default", "aten.flatten.using_ints",
                  "aten.unsqueeze.default", "aten.squeeze.dim"):
            r = V.try_reshape(v, out.shape)
            if r is None:
                src = self.contiguous(src)
                r = V.try_reshape(self.view(src), out.shape)
            return self.alias(node, src, r)
        if op == "aten.t.default":
            return self.alias(node, src, V.transpose(v, 0, 1) if nd == 2 else v)
        if op == "aten.transpose.int":
            return self.alias(node, src, V.transpose(v, a.get("dim0", 0), a.get("dim1", 1)))
        if op == "aten.permute.default":
            return self.alias(node, src, V.permute(v, a.get("dims")))
        if op == "aten.expand.default":
            return self.alias(node, src, V.broadcast_to(v, out.shape))
        if op == "aten.slice.Tensor":
            return self.alias(node, src, V.slice_(v, a.get("dim", 0), a.get("start"), a.get("end"), a.get("step", 1)))
        raise ValueError(f"Unknown alias op: {op}")

    def lower_cat(self, node: OpNode) -> None:
        out = node.outputs[0]
        parts = [t for t in node.inputs if list(t.shape) != [0]]
        if len(parts) == 1 and list(parts[0].shape) == list(out.shape):
            return self.alias(node, parts[0].name, self.view(parts[0].name))
        nd = len(out.shape)
        dim = node.attrs.get("dim", 0)
        dim = dim + nd if dim < 0 else dim
        dst = self.alloc(out.name, out.shape, self.sd(out.dtype))
        at = 0
        for i, t in enumerate(parts):
            ext = t.shape[dim]
            piece = V.slice_(dst, dim, at, at + ext, 1)
            pname = f"{out.name}__part{i}"
            self.out.views[pname] = piece
            self.emit(SpecialKernelStep("strided_copy", "cat piece", [t.name], out.name,
                                        params={"op": "strided_copy", "in_view": self.view(t.name), "out_view": piece}),
                      [t.name, out.name])
            at += ext

    # -- elementwise chains -----------------------------------------------------------
    def _chain_member(self, node: OpNode) -> bool:
        if node.op_type in ("aten.to.dtype", "aten._to_copy.default"):
            return True
        return is_fusible_elementwise(node.op_type) and not node.op_type.startswith("b200.")

    def lower_chain(self, first: OpNode) -> None:
        """Greedy chain: follow the single consumer while it is elementwise, keeps the
        output shape and stays within the operand/op limits (reference:
        subgraph_analyzer.py:984-1044)."""
        chain = [first]
        shape = list(first.outputs[0].shape)
        cur = first
        while self.fuse and len(chain) < MAX_CHAIN_OPS:
            nxt = self.gi.sole_consumer(cur.outputs[0].name)
            if nxt is None or id(nxt) in self._chain_done or not self._chain_member(nxt):
                break
            if self.gi.position[id(nxt)] != self.gi.position[id(cur)] + 1 and not self._inputs_ready(nxt, chain):
                break
            if list(nxt.outputs[0].shape) != shape:
                break
            if nxt.op_type in ("aten.to.dtype", "aten._to_copy.default") and self.sd(nxt.outputs[0].dtype) == self.sd(cur.outputs[0].dtype):
                break  # a no-op cast is an alias; leave it to the alias path
            if len(self._chain_inputs(chain + [nxt])) > MAX_CHAIN_INPUTS:
                break
            chain.append(nxt)
            cur = nxt
        ext_inputs = self._chain_inputs(chain)
        if len(ext_inputs) > MAX_CHAIN_INPUTS:
            raise ValueError(f"elementwise op {first.name} has too many tensor operands")
        slot = {name: i for i, name in enumerate(ext_inputs)}
        program = []
        for j, n in enumerate(chain):
            program.append(self._encode(n, slot))
            slot[n.outputs[0].name] = MAX_CHAIN_INPUTS + j
        last = chain[-1].outputs[0]
        like = next((n for n in ext_inputs if tuple(self.view(n).shape) == tuple(last.shape)), None)
        out_view = self.out_like(last, like)
        in_views = [V.broadcast_to(self._pad_rank(self.view(n), len(last.shape)), last.shape) for n in ext_inputs]
        for n in chain[1:]:
            self._chain_done.add(id(n))
        kname = "fused_" + "_".join(n.op_type.split(".")[1].rstrip("_") for n in chain)
        self.emit(FusedKernelStep(kernel_name=kname, source_code=describe_chain(chain), input_buffer_names=list(ext_inputs),
                                  output_buffer_name=last.name, total_elements=int(math.prod(last.shape)),
                                  params={"op": "ew_chain", "in_views": in_views, "out_view": out_view, "program": program}),
                  list(ext_inputs) + [last.name])

    def _inputs_ready(self, nxt: OpNode, chain: list[OpNode]) -> bool:
        """A later chain member may be pulled up to the chain head only if its other
        operands are already defined there."""
        head = self.gi.position[id(chain[0])]
        inside = {n.outputs[0].name for n in chain}
        for t in nxt.inputs:
            if t.name in inside:
                continue
            p = self.gi.producer.get(t.name)
            if p is not None and self.gi.position[id(p)] > head:
                return False
        # and nothing between head and nxt may read what nxt overwrites: outputs are fresh names, so safe
        return True

    @staticmethod
    def _pad_rank(v: TensorView, nd: int) -> TensorView:
        while len(v.shape) < nd:
            v = V.unsqueeze(v, 0)
        return v

    def _chain_inputs(self, chain: list[OpNode]) -> list[str]:
        inside = {n.outputs[0].name for n in chain}
        names: list[str] = []
        for n in chain:
            for t in n.inputs:
                if t.name not in inside and t.name not in names:
                    names.append(t.name)
        return names

    def _encode(self, n: OpNode, slot: dict[str, int]) -> tuple:
        op = n.op_type
        rd = self.sd(n.outputs[0].dtype)
        if op in ("aten.to.dtype", "aten._to_copy.default"):
            return ("CAST", slot[n.inputs[0].name], -1, rd, 0.0)
        base = op.split(".")[1].rstrip("_")
        a = slot[n.inputs[0].name]
        if base in ("add", "sub", "mul", "div"):
            if n.attrs.get("alpha", 1) not in (1, 1.0, None):
                raise ValueError(f"{op} with alpha != 1 is not supported")
            if len(n.inputs) == 2:
                return (base.upper(), a, slot[n.inputs[1].name], rd, 0.0)
            other = n.attrs.get("other")
            if not isinstance(other, (int, float)):
                raise ValueError(f"{op} node {n.name} has neither a second tensor nor a scalar 'other'")
            return (base.upper() + "_S", a, -1, rd, float(other))
        if base == "pow":
            return ("POW_S", a, -1, rd, float(n.attrs.get("exponent", 2)))
        if base.upper() in EW_OPCODES:
            return (base.upper(), a, -1, rd, 0.0)
        raise ValueError(f"Unknown elementwise op: {op}")

    # -- reductions ------------------------------------------------------------------
    def lower_reduction(self, node: OpNode) -> None:
        op, a = node.op_type, node.attrs
        out = node.outputs[0]
        x = node.inputs[0].name
        if op in ("aten.softmax.int", "aten._softmax.default"):
            return self._softmax(node, x, None, 1.0, out, node.inputs[0].dtype)
        if op == "aten.mean.dim":
            v = self.view(x)
            nd = len(v.shape)
            dims = a.get("dim", [-1])
            dims = sorted(d + nd if d < 0 else d for d in ([dims] if isinstance(dims, int) else dims))
            if dims == [nd - 1]:
                xc = self.contiguous(x)
                cols = v.shape[-1]
                o = self.alloc(out.name, out.shape, self.sd(out.dtype))
                return self.emit(ReductionKernelStep("mean_last_dim_kernel", "mean over last axis", [xc], out.name,
                                                     params={"op": "mean_last_dim", "rows": v.numel // cols, "cols": cols,
                                                             "x": self.view(xc), "y": o}), [xc, out.name])
            if nd == 4 and dims == [2, 3]:
                o = self.alloc(out.name, out.shape, self.sd(out.dtype))
                N, C = v.shape[:2]
                y4 = TensorView(o.buffer, 0, (N, C, 1, 1), (C, 1, 1, 1), o.dtype)
                return self.emit(ReductionKernelStep("adaptive_avg_pool2d_kernel", "global average pool", [x], out.name,
                                                     params={"op": "adaptive_avg_pool2d", "x": v, "y": y4, "batch": N, "channels": C}),
                                 [x, out.name])
            raise ValueError(f"mean over dims {dims} is not supported")
        if op == "aten.max_pool2d.default":
            k = a.get("kernel_size", [2, 2])
            k = [k, k] if isinstance(k, int) else list(k)
            s = a.get("stride") or k
            s = [s, s] if isinstance(s, int) else list(s)
            p = a.get("padding", [0, 0])
            p = [p, p] if isinstance(p, int) else list(p)
            d = a.get("dilation", [1, 1])
            if (d not in (1, [1, 1], [1])) or a.get("ceil_mode", False):
                raise ValueError("max_pool2d with dilation/ceil_mode is not supported")
            o = self.out_like_nchw(out, x)
            v = self.view(x)
            return self.emit(ReductionKernelStep("max_pool2d_kernel", "max pool", [x], out.name,
                                                 params={"op": "max_pool2d", "x": v, "y": o, "kernel_h": k[0], "kernel_w": k[-1],
                                                         "stride_h": s[0], "stride_w": s[-1], "pad_h": p[0], "pad_w": p[-1],
                                                         "batch": v.shape[0], "channels": v.shape[1]}), [x, out.name])
        if op == "aten.adaptive_avg_pool2d.default":
            o = self.out_like_nchw(out, x)
            v = self.view(x)
            return self.emit(ReductionKernelStep("adaptive_avg_pool2d_kernel", "adaptive average pool", [x], out.name,
                                                 params={"op": "adaptive_avg_pool2d", "x": v, "y": o, "batch": v.shape[0],
                                                         "channels": v.shape[1]}), [x, out.name])
        if op == "aten.batch_norm.default":
            if a.get("training", False):
                raise ValueError("batch_norm in training mode is not supported")
            names = self._optional_operands(node, ["weight", "bias", "running_mean", "running_var"])
            if names["running_mean"] is None or names["running_var"] is None:
                raise ValueError("batch_norm without running statistics is not supported")
            o = self.out_like_nchw(out, x)
            v = self.view(x)
            if len(v.shape) != 4:
                raise ValueError("batch_norm is implemented for 4-D inputs")
            ins = [x] + [n for n in names.values() if n is not None]
            return self.emit(ReductionKernelStep("batch_norm_kernel", "inference batch-norm", ins, out.name,
                                                 params={"op": "batch_norm", "x": v, "y": o, "gamma": names["weight"],
                                                         "beta": names["bias"], "mean": names["running_mean"],
                                                         "var": names["running_var"], "eps": float(a.get("eps", 1e-5)),
                                                         "relu": False, "batch": v.shape[0], "channels": v.shape[1]}),
                             ins + [out.name])
        if op == "aten.argmax.default":
            v = self.view(x)
            nd = len(v.shape)
            dim = a.get("dim")
            if dim is None or (dim + nd if dim < 0 else dim) != nd - 1:
                raise ValueError("argmax is implemented over the last axis only")
            xc = self.contiguous(x)
            o = self.alloc(out.name, out.shape, "int64")
            cols = v.shape[-1]
            return self.emit(ReductionKernelStep("argmax_rows_kernel", "argmax over last axis", [xc], out.name,
                                                 params={"op": "argmax", "x": self.view(xc), "y": o, "rows": v.numel // cols,
                                                         "cols": cols}), [xc, out.name])
        raise ValueError(f"Unknown reduction op: {op}")

    def out_like_nchw(self, out: TensorSpec, like: str) -> TensorView:
        v = self.view(like)
        shape = tuple(out.shape)
        if len(shape) == 4 and len(v.shape) == 4 and v.strides[1] == 1 and v.shape[1] > 1:  # channels-last stays channels-last
            N, C, H, W = shape
            return self.alloc(out.name, shape, self.sd(out.dtype), (H * W * C, 1, W * C, C))
        return self.alloc(out.name, shape, self.sd(out.dtype))

    def _optional_operands(self, node: OpNode, names: list[str]) -> dict[str, str | None]:
        """Tensor operands after the first, some of which may be absent (then the
        exporter stored ``None`` under the argument's name in attrs)."""
        rest = [t.name for t in node.inputs[1:]]
        result: dict[str, str | None] = {}
        for n in names:
            if n in node.attrs and node.attrs[n] is None:
                result[n] = None
            else:
                result[n] = rest.pop(0) if rest else None
        return result

    def _softmax(self, node, x: str, mask: str | None, scale: float, out: TensorSpec, sum_dtype: str) -> None:
        xc = self.contiguous(x)
        v = self.view(xc)
        nd = len(v.shape)
        shape4 = (1,) * (4 - nd) + tuple(v.shape) if nd <= 4 else (math.prod(v.shape[:-3]),) + tuple(v.shape[-3:])
        ms = (0, 0, 0)
        ins = [xc]
        mview = None
        if mask is not None:
            if nd > 4:
                raise ValueError("masked softmax over more than 4 dims")
            mview = V.broadcast_to(self._pad_rank(self.view(mask), nd), v.shape)
            mview = self._pad_rank(mview, 4)
            if mview.strides[3] != 1 and mview.shape[3] > 1:
                mc = self.contiguous(mask)
                mview = self._pad_rank(V.broadcast_to(self._pad_rank(self.view(mc), nd), v.shape), 4)
                mask = mc
            ms = tuple(mview.strides[:3])
            ins.append(mask)
        o = self.alloc(out.name, out.shape, self.sd(out.dtype))
        name = "masked_softmax_kernel" if mask is not None else "softmax_kernel"
        self.emit(ReductionKernelStep(name, "softmax(x*scale + mask) over last axis", ins, out.name,
                                      params={"op": "softmax", "x": v, "mask": mview, "y": o, "rows": v.numel // v.shape[-1],
                                              "cols": v.shape[-1], "dims": shape4[:3], "mask_strides": ms, "scale": scale,
                                              "round_steps": self.sd(sum_dtype) != "float32"}),
                  ins + [out.name])

    def lower_softmax(self, node: OpNode) -> None:  # b200.softmax macro
        scores, mask = node.inputs
        self._softmax(node, scores.name, mask.name, node.attrs["scale"], node.outputs[0], node.attrs["sum_dtype"])

    def lower_rmsnorm(self, node: OpNode) -> None:
        x, w = node.inputs
        out = node.outputs[0]
        dt = self.sd(out.dtype)
        if dt not in ("float16", "bfloat16") or self.view(x.name).dtype != dt:
            return self.lower_original(node)
        xn, x2 = self.as_2d(x.name)
        o = self.alloc(out.name, out.shape, dt)
        rows, cols = x2.shape
        self.emit(ReductionKernelStep("rmsnorm_kernel", "x * rsqrt(mean(x^2) + eps) * w", [xn, w.name], out.name,
                                      params={"op": "rmsnorm", "x": x2, "w": w.name, "y": o, "rows": rows, "cols": cols,
                                              "eps": node.attrs["eps"], "round_mid": node.attrs["round_mid"]}),
                  [xn, w.name, out.name])

    def lower_original(self, node: OpNode) -> None:
        """A fused pattern that cannot use its kernel falls back to its own nodes."""
        for n in node.attrs["_orig"]:
            if id(n) not in self._chain_done:
                self.lower(n)

    # -- special ops ---------------------------------------------------------------------
    def lower_special(self, node: OpNode) -> None:
        op, a = node.op_type, node.attrs
        out = node.outputs[0] if node.outputs else None
        if op == "aten.embedding.default":
            table, ids = node.inputs[0].name, node.inputs[1].name
            idc = self.contiguous(ids)
            tv = self.view(table)
            o = self.alloc(out.name, out.shape, tv.dtype)
            n_ids = self.view(idc).numel
            return self.emit(SpecialKernelStep("embedding_kernel", "out[s,:] = table[ids[s],:]", [idc, table], out.name,
                                               params={"op": "embedding", "table": table, "ids": self.view(idc), "y": o,
                                                       "seq_len": n_ids, "embed_dim": tv.shape[1], "vocab": tv.shape[0]},
                                               grid_dim=(1, n_ids)), [idc, table, out.name])
        if op == "wrap_with_set_grad_enabled":
            inv, pos = node.inputs[0].name, node.inputs[1].name
            pc = self.contiguous(pos)
            cos, sin = node.outputs[0], node.outputs[1]
            dt = self.sd(cos.dtype)
            oc = self.alloc(cos.name, cos.shape, dt)
            os_ = self.alloc(sin.name, sin.shape, dt)
            hd = cos.shape[-1]
            n_pos = self.view(pc).numel
            return self.emit(SpecialKernelStep("rope_kernel", "cos/sin(position * inv_freq)", [inv, pc], cos.name,
                                               output_buffer_names=[cos.name, sin.name],
                                               params={"op": "rope_table", "inv_freq": inv, "pos": self.view(pc), "cos": oc, "sin": os_,
                                                       "seq_len": n_pos, "head_dim": hd}, grid_dim=(1, n_pos)),
                             [inv, pc, cos.name, sin.name])
        if op == "aten.index_copy.default":
            return self.lower_index_copy(node)
        if op == "aten.full.default":
            o = self.alloc(out.name, out.shape, self.sd(out.dtype))
            return self.emit(SpecialKernelStep("full_kernel", "fill", [], out.name,
                                               params={"op": "fill", "y": o, "fill_value": float(a.get("fill_value", 0.0)),
                                                       "total": o.numel}), [out.name])
        raise ValueError(f"Unknown special op: {op}")

    def lower_index_copy(self, node: OpNode, src_override: str | None = None) -> None:
        base, index, src = node.inputs[0].name, node.inputs[1].name, src_override or node.inputs[2].name
        out = node.outputs[0]
        bv = self.view(base)
        nd = len(bv.shape)
        dim = node.attrs.get("dim", 0)
        dim = dim + nd if dim < 0 else dim
        if not bv.is_contiguous():
            base = self.contiguous(base)
            bv = self.view(base)
        outer, dim_size, inner = math.prod(bv.shape[:dim]), bv.shape[dim], math.prod(bv.shape[dim + 1:])
        sv = self.view(src)
        n_index = sv.shape[dim]
        s3 = None
        if sv.dtype == bv.dtype:
            # need src as [outer, n_index, inner] with inner contiguous
            perm = V.try_reshape(sv, (outer, n_index, inner)) if outer * n_index * inner == sv.numel else None
            if perm is not None and (perm.strides[2] == 1 or inner == 1):
                s3 = perm
        if s3 is None:
            if sv.dtype != bv.dtype:
                raise ValueError("index_copy source dtype differs from destination")
            src = self.contiguous(src)
            s3 = V.try_reshape(self.view(src), (outer, n_index, inner))
        idx = self.contiguous(index)
        in_place = (self.donate and base in self.external and base not in self.weight_names and base not in self.keep_inputs
                    and len(self.gi.consumers.get(base, [])) == 1)
        if in_place:
            self.out.views[out.name] = TensorView(bv.buffer, bv.offset, tuple(out.shape), V.contiguous_strides(out.shape), bv.dtype)
            self.out.donated[out.name] = base
            o = self.out.views[out.name]
        else:
            o = self.alloc(out.name, out.shape, bv.dtype)
        self.emit(SpecialKernelStep("index_copy_kernel", "dst[..., index[l], :] = src[..., l, :]" + (" (in place)" if in_place else ""),
                                    [base, src, idx], out.name,
                                    params={"op": "index_copy", "base": bv, "dst": o, "src": s3, "index": self.view(idx),
                                            "outer_size": outer, "dim_size": dim_size, "inner_size": inner,
                                            "num_indices": n_index, "in_place": in_place}),
                  [base, src, idx, out.name])

    def lower_rope_rotate(self, node: OpNode) -> None:
        x, cos_u, sin_u = node.inputs
        out = node.outputs[0]
        xv, cv, sv = self.view(x.name), self.view(cos_u.name), self.view(sin_u.name)
        B, H, T, D = xv.shape
        dt = self.sd(out.dtype)

        def table_ok(v: TensorView) -> bool:  # [B,1,T,D] dense over (b, t, d)
            return v.dtype == dt and v.strides[3] == 1 and (T == 1 or v.strides[2] == D) and (B == 1 or v.strides[0] == T * D)

        if dt not in ("float16", "bfloat16") or xv.dtype != dt or xv.strides[3] != 1 or not table_ok(cv) or not table_ok(sv) \
                or any(s % 8 for s in xv.strides[:3]) or xv.offset % 8 or cv.offset % 8 or sv.offset % 8:
            return self.lower_original(node)
        o = self.alloc(out.name, out.shape, dt)
        self.emit(SpecialKernelStep("rope_rotate_kernel", "x*cos + rotate_half(x)*sin", [x.name, cos_u.name, sin_u.name], out.name,
                                    params={"op": "rope_rotate", "x": xv, "cos": cv, "sin": sv, "y": o}),
                  [x.name, cos_u.name, sin_u.name, out.name])

    def lower_rope_pair(self, node: OpNode) -> None:
        q, k, cos_u, sin_u = node.inputs
        q_out, k_out = node.outputs
        qv, kv, cv, sv = (self.view(t.name) for t in (q, k, cos_u, sin_u))
        B, _, T, D = qv.shape
        dt = self.sd(q_out.dtype)

        def table_ok(v: TensorView) -> bool:  # [B,1,T,D] dense over (b, t, d)
            return v.dtype == dt and v.strides[3] == 1 and (T == 1 or v.strides[2] == D) and (B == 1 or v.strides[0] == T * D) and v.offset % 8 == 0

        ok = dt in ("float16", "bfloat16") and self.sd(k_out.dtype) == dt and D % 16 == 0 and table_ok(cv) and table_ok(sv)
        ok = ok and all(t.dtype == dt and t.strides[3] == 1 and t.offset % 8 == 0 and all(s % 8 == 0 for s in t.strides[:3]) for t in (qv, kv))
        if not ok:
            return self.lower_original(node)
        qo = self.alloc(q_out.name, q_out.shape, dt)
        ko = self.alloc(k_out.name, k_out.shape, dt)
        names = [q.name, k.name, cos_u.name, sin_u.name]
        self.emit(SpecialKernelStep("rope_rotate_pair_kernel", "q*cos + rotate_half(q)*sin; k*cos + rotate_half(k)*sin", names, q_out.name,
                                    output_buffer_names=[q_out.name, k_out.name],
                                    params={"op": "rope_rotate_pair", "q": qv, "k": kv, "cos": cv, "sin": sv, "q_out": qo, "k_out": ko}),
                  names + [q_out.name, k_out.name])

    def lower_qkv_post(self, node: OpNode) -> None:
        q, k, v, cos_u, sin_u, cache_k, cache_v, index = node.inputs
        q_out, kc_out, vc_out = node.outputs
        dt = self.sd(q_out.dtype)
        views = [self.view(t.name) for t in (q, k, v)]
        cv, sv = self.view(cos_u.name), self.view(sin_u.name)
        B, Hq, T, D = views[0].shape

        def table_ok(t: TensorView) -> bool:
            return t.dtype == dt and t.strides[3] == 1 and (T == 1 or t.strides[2] == D) and (B == 1 or t.strides[0] == T * D) and t.offset % 8 == 0

        def donatable(c) -> bool:
            cvw = self.view(c.name)
            return (self.donate and c.name in self.external and c.name not in self.weight_names and c.name not in self.keep_inputs
                    and cvw.is_contiguous() and cvw.dtype == dt and len(self.gi.consumers.get(c.name, [])) == 1)

        ok = dt in ("float16", "bfloat16") and D % 16 == 0 and table_ok(cv) and table_ok(sv) and donatable(cache_k) and donatable(cache_v)
        ok = ok and all(t.dtype == dt and t.strides[3] == 1 and t.offset % 8 == 0 and all(s % 8 == 0 for s in t.strides[:3]) for t in views)
        if not ok:
            return self.lower_original(node)
        idx = self.contiguous(index.name)
        qo = self.alloc(q_out.name, q_out.shape, dt)
        for c, o in ((cache_k, kc_out), (cache_v, vc_out)):
            base = self.view(c.name)
            self.out.views[o.name] = TensorView(base.buffer, base.offset, tuple(o.shape), V.contiguous_strides(o.shape), base.dtype)
            self.out.donated[o.name] = c.name
        names = [t.name for t in (q, k, v, cos_u, sin_u, cache_k, cache_v)] + [idx]
        self.emit(SpecialKernelStep("qkv_rope_cache_kernel", "rope(q); key cache[pos] = rope(k); value cache[pos] = v  (in place)",
                                    names, q_out.name, output_buffer_names=[q_out.name, kc_out.name, vc_out.name],
                                    params={"op": "qkv_post", "q": views[0], "k": views[1], "v": views[2], "cos": cv, "sin": sv, "q_out": qo,
                                            "k_cache": self.view(cache_k.name), "v_cache": self.view(cache_v.name), "index": self.view(idx),
                                            "cache_len": cache_k.shape[2], "in_place": True}),
                  names + [q_out.name, kc_out.name, vc_out.name])

    # -- dense contractions -----------------------------------------------------------------
    def lower_blas(self, node: OpNode) -> None:
        op = node.op_type
        if op == "aten.linear.default":
            return self._linear(node, node.inputs, node.outputs[0], has_bias=len(node.inputs) > 2)
        if op == "aten.conv2d.default":
            attrs = {k: node.attrs.get(k) for k in ("stride", "padding", "dilation", "groups")}
            attrs.update(has_bias=len(node.inputs) > 2, bn=False, residual=False, relu=False, eps=0.0)
            return self.lower_conv2d(OpNode(node.name, "b200.conv2d", list(node.inputs), list(node.outputs), attrs))
        if op in ("aten.matmul.default", "aten.mm.default", "aten.bmm.default"):
            return self._matmul(node.inputs[0].name, node.inputs[1].name, node.outputs[0])
        if op == "aten.addmm.default":
            bias, x, w = node.inputs
            tmp = TensorSpec(node.outputs[0].name + "__mm", node.outputs[0].shape, node.outputs[0].dtype)
            self._matmul(x.name, w.name, tmp)
            out = node.outputs[0]
            o = self.alloc(out.name, out.shape, self.sd(out.dtype))
            ins = [tmp.name, bias.name]
            in_views = [V.broadcast_to(self._pad_rank(self.view(n), len(out.shape)), out.shape) for n in ins]
            return self.emit(FusedKernelStep("fused_add", "mm + bias", ins, out.name, int(math.prod(out.shape)),
                                             params={"op": "ew_chain", "in_views": in_views, "out_view": o,
                                                     "program": [("ADD", 0, 1, o.dtype, 0.0)]}), ins + [out.name])
        raise ValueError(f"Unknown BLAS op: {op}")

    def lower_linear(self, node: OpNode) -> None:  # b200.linear macro
        a = node.attrs
        if a.get("glu"):
            return self._linear_glu(node)
        n_base = 3 if a["has_bias"] else 2
        extra = list(node.inputs[n_base:])
        residual = extra.pop(0) if a["residual"] else None
        aux = extra.pop(0) if a["silu_mul"] else None
        self._linear(node, node.inputs[:n_base], node.outputs[0], has_bias=a["has_bias"], residual=residual, aux=aux,
                     relu=a["relu"])

    def lower_linear_group(self, node: OpNode) -> None:
        """q/k/v-style projections of one activation as a single GEMM over concatenated weights."""
        a = node.attrs
        per = 2 if a["has_bias"] else 1
        x = node.inputs[0]
        ws = [node.inputs[1 + per * i] for i in range(a["n_parts"])]
        bs = [node.inputs[2 + per * i] for i in range(a["n_parts"])] if a["has_bias"] else []
        outs = node.outputs
        dt = self.sd(outs[0].dtype)
        if dt not in ("float16", "bfloat16") or self.view(x.name).dtype != dt:
            return self.lower_original(node)
        rows = [int(w.shape[0]) for w in ws]
        K, n_total = int(ws[0].shape[1]), sum(rows)
        wp, bp = f"{node.name}__w", f"{node.name}__b"
        self.out.weight_preps.append(WeightPrep("concat_rows", [w.name for w in ws], [wp], {"rows": rows, "cols": K, "dtype": dt}))
        self.out.views[wp] = TensorView(wp, 0, (n_total, K), (K, 1), dt)
        if bs:
            self.out.weight_preps.append(WeightPrep("concat_rows", [b.name for b in bs], [bp], {"rows": rows, "cols": 1, "dtype": dt}))
            self.out.views[bp] = TensorView(bp, 0, (n_total,), (1,), dt)
        merged = TensorSpec(f"{node.name}__out", list(outs[0].shape[:-1]) + [n_total], outs[0].dtype)
        fake_ins = [x, TensorSpec(wp, [n_total, K], ws[0].dtype)] + ([TensorSpec(bp, [n_total], bs[0].dtype)] if bs else [])
        self._linear(node, fake_ins, merged, has_bias=bool(bs))
        full = self.view(merged.name)
        nd = len(full.shape)
        at = 0
        for o, n in zip(outs, rows):
            self.out.views[o.name] = V.slice_(full, nd - 1, at, at + n, 1)
            self.emit(AliasStep(merged.name, o.name, list(full.shape), list(o.shape)), [merged.name, o.name])
            at += n

    def _linear_glu(self, node: OpNode) -> None:
        """silu(x Wg^T) * (x Wu^T) as one GEMM over gate/up rows interleaved in blocks of 64."""
        x, wg, wu = node.inputs
        out = node.outputs[0]
        dt = self.sd(out.dtype)
        inter, K = int(wg.shape[0]), int(wg.shape[1])
        if dt not in ("float16", "bfloat16") or self.view(x.name).dtype != dt or K % 8:
            return self.lower_original(node)
        wp = f"{node.name}__w"
        self.out.weight_preps.append(WeightPrep("interleave_rows", [wg.name, wu.name], [wp], {"rows": inter, "cols": K, "block": 64, "dtype": dt}))
        self.out.views[wp] = TensorView(wp, 0, (2 * inter, K), (K, 1), dt)
        self._linear(node, [x, TensorSpec(wp, [2 * inter, K], wg.dtype)], out, has_bias=False, glu=True)

    def _linear(self, node, ins, out: TensorSpec, has_bias: bool, residual=None, aux=None, relu=False, glu=False) -> None:
        x, w = ins[0].name, ins[1].name
        bias = ins[2].name if has_bias else None
        dt = self.sd(out.dtype)
        if dt not in ("float16", "bfloat16"):
            raise ValueError(f"linear in {dt} is not supported: compile with compute_dtype float16 or bfloat16")
        xv = self.view(x)
        if xv.dtype != dt:
            raise ValueError(f"linear input {x} is {xv.dtype}, expected {dt}")
        xn, x2 = self.as_2d(x)
        M, K = x2.shape
        N = self.view(w).shape[0]          # rows of W (gate and up rows together for the gated form)
        n_out = N // 2 if glu else N
        if x2.strides[0] % 8 or x2.offset % 8:
            xn = self.contiguous(xn, "aligned")
            x2 = V.try_reshape(self.view(xn), (M, K))
        o = self.alloc(out.name, out.shape, dt)
        o2 = V.try_reshape(o, (M, n_out))
        names = [xn, w]
        p = {"op": "linear", "x": x2, "w": w, "bias": bias, "y": o2, "M": M, "N": N, "K": K, "transpose_b": True,
             "has_bias": has_bias, "relu": bool(relu), "residual": None, "aux": None, "workspace": None, "glu": bool(glu)}
        if bias:
            names.append(bias)
        for key, t in (("residual", residual), ("aux", aux)):
            if t is not None:
                tn, t2 = self.as_2d(t.name)
                if t2.dtype != dt:
                    raise ValueError(f"linear epilogue operand {t.name} has dtype {t2.dtype}, expected {dt}")
                p[key] = t2
                names.append(tn)
        # split-K scratch (sized by the library for the largest (M, N, K) of the program; shared, self-cleaning)
        p["workspace"] = "__ws_splitk"
        names.append("__ws_splitk")
        self.out.buffers.setdefault("__ws_splitk", BufferAllocation("__ws_splitk", [0], "uint8", 0, persistent=True))
        p["workspace_key"] = (M, N, K)
        desc = "x @ W^T" + (" + b" if has_bias else "") + (" + residual" if residual is not None else "") + \
               (" -> relu" if relu else "") + (" -> silu(.) * up" if aux is not None else "") + (" -> silu(gate) * up, interleaved rows" if glu else "")
        self.emit(CUBLASStep("gemm", names, out.name, p), names + [out.name])
        self.out.steps[-1].params["source"] = desc

    def _matmul(self, a: str, b: str, out: TensorSpec) -> None:
        av, bv = self.view(a), self.view(b)
        dt = self.sd(out.dtype)
        if av.dtype != dt or bv.dtype != dt:
            raise ValueError("matmul operands must share the output dtype")
        if len(av.shape) == 1 or len(bv.shape) == 1:
            raise ValueError("matmul with 1-D operands is not supported")
        M, K, N = av.shape[-2], av.shape[-1], bv.shape[-1]
        batch = tuple(out.shape[:-2])
        if len(batch) > 2:
            raise ValueError("matmul with more than two batch dims is not supported")
        b2 = (1,) * (2 - len(batch)) + batch
        full = lambda v, tail: self._pad_rank(V.broadcast_to(self._pad_rank(v, len(batch) + 2), batch + tail), 4)
        a4, b4 = full(av, (M, K)), full(bv, (K, N))
        o = self.alloc(out.name, out.shape, dt)
        o4 = self._pad_rank(o, 4)
        blas_type = "gemm_batched" if batch else "gemm"
        self.emit(CUBLASStep(blas_type, [a, b], out.name,
                             {"op": "matmul", "a": a4, "b": b4, "y": o4, "batch": math.prod(b2), "b1": b2[0], "b2": b2[1], "M": M, "N": N,
                              "K": K, "transpose_b": False, "has_bias": False}), [a, b, out.name])

    def lower_conv2d(self, node: OpNode) -> None:  # b200.conv2d macro (also plain conv)
        a = node.attrs
        ins = list(node.inputs)
        x, w = ins[0], ins[1]
        rest = ins[2:]
        conv_bias = rest.pop(0).name if a["has_bias"] else None
        bn = [rest.pop(0).name for _ in range(4)] if a["bn"] else [None] * 4
        residual = rest.pop(0) if a["residual"] else None
        out = node.outputs[0]
        dt = self.sd(out.dtype)
        if dt not in ("float16", "bfloat16"):
            raise ValueError(f"conv2d in {dt} is not supported: compile with compute_dtype float16 or bfloat16")

        def pair(v, default):
            v = default if v is None else v
            return [v, v] if isinstance(v, int) else list(v)

        stride, pad, dil = pair(a.get("stride"), 1), pair(a.get("padding"), 0), pair(a.get("dilation"), 1)
        if (a.get("groups") or 1) != 1 or dil != [1, 1]:
            raise ValueError("conv2d with groups != 1 or dilation != 1 is not supported")
        N, C, H, W = x.shape
        O, _, KH, KW = w.shape
        Ho, Wo = out.shape[2], out.shape[3]
        Cp = (C + 7) // 8 * 8
        xv = self.view(x.name)
        xin = x.name
        nhwc = (H * W * Cp, 1, W * Cp, Cp)
        if not (xv.dtype == dt and C == Cp and tuple(xv.strides) == nhwc and xv.offset % 8 == 0):
            # repack to channels-last with channels padded to a multiple of 8 (padding stays zero)
            xin = f"{x.name}__nhwc{Cp}"
            if xin not in self.out.views:
                full = self.alloc(xin, (N, Cp, H, W), dt, nhwc, persistent=Cp != C)
                piece = V.slice_(full, 1, 0, C, 1)
                self.emit(SpecialKernelStep("strided_copy", "NCHW -> NHWC repack", [x.name], xin,
                                            params={"op": "strided_copy", "in_view": xv, "out_view": piece}), [x.name, xin])
        wp, bp = f"{node.name}__w", f"{node.name}__bias"
        self.out.weight_preps.append(WeightPrep("conv_fold", [w.name, conv_bias] + bn, [wp, bp],
                                                {"O": O, "I": C, "KH": KH, "KW": KW, "I_pad": Cp, "eps": a["eps"], "dtype": dt}))
        o = self.alloc(out.name, out.shape, dt, (Ho * Wo * O, 1, Wo * O, O))
        names = [xin]
        res_view = None
        if residual is not None:
            rv = self.view(residual.name)
            rn = residual.name
            if not (rv.dtype == dt and tuple(rv.strides) == tuple(o.strides) and rv.offset % 2 == 0):
                rn = f"{residual.name}__nhwc"
                if rn not in self.out.views:
                    self.alloc(rn, rv.shape, dt, o.strides)
                    self.copy(residual.name, rn)
            res_view = self.view(rn)
            names.append(rn)
        self.emit(CUBLASStep("conv2d", names + [w.name], out.name,
                             {"op": "conv2d", "x": self.view(xin), "w_prepared": wp, "bias_prepared": bp, "residual": res_view, "y": o,
                              "batch": N, "in_channels": C, "in_h": H, "in_w": W, "out_channels": O, "out_h": Ho, "out_w": Wo,
                              "kernel_h": KH, "kernel_w": KW, "stride_h": stride[0], "stride_w": stride[1], "pad_h": pad[0],
                              "pad_w": pad[1], "has_bias": a["has_bias"], "groups": 1, "c_pad": Cp, "relu": a["relu"],
                              "bn_folded": a["bn"]}), names + [out.name])

    def lower_attention(self, node: OpNode) -> None:
        a = node.attrs
        q, k, v = node.inputs[:3]
        mask = node.inputs[3] if a["has_mask"] else None
        out = node.outputs[0]
        dt = self.sd(out.dtype)
        qv, kv, vv = self.view(q.name), self.view(k.name), self.view(v.name)
        B, Hq, Hkv, T, S, D = a["B"], a["Hq"], a["Hkv"], a["T"], a["S"], a["D"]
        ok = dt in ("float16", "bfloat16") and all(t.dtype == dt and t.strides[3] == 1 and t.offset % 8 == 0 and
                                                   all(s % 8 == 0 for s in t.strides[:3]) for t in (qv, kv, vv))
        mv = None
        if ok and mask is not None:
            mv = V.broadcast_to(self.view(mask.name), (B, 1, T, S))
            ok = mv.dtype == dt and (mv.strides[3] == 1 or S == 1)
        if ok and T == 1:
            # decode kernel wants q as [B, Hq*D] rows and dense [S, D] planes per (b, kv head)
            ok = qv.strides[1] == D and kv.strides[2] == D and vv.strides[2] == D and tuple(kv.strides) == tuple(vv.strides)
        if not ok:
            return self.lower_original(node)
        o = self.alloc(out.name, out.shape, dt)
        names = [q.name, k.name, v.name] + ([mask.name] if mask is not None else [])
        p = {"op": "attention", "q": qv, "k": kv, "v": vv, "mask": mv, "y": o, "scale": a["scale"], "B": B, "Hq": Hq, "Hkv": Hkv,
             "T": T, "S": S, "D": D, "decode": T == 1, "workspace": None}
        if T == 1:
            p["workspace"] = "__ws_attn"
            names.append("__ws_attn")
            self.out.buffers.setdefault("__ws_attn", BufferAllocation("__ws_attn", [0], "uint8", 0, persistent=True))
        self.emit(CUBLASStep("attention", names, out.name, p), names + [out.name])


def analyze(graph: IRGraph, compute_dtype: str | None = None, donate: bool = True, fuse: bool = True, keep_inputs=()) -> Analysis:
    cd = infer_compute_dtype(graph, compute_dtype)
    return _Lowering(graph, cd, donate=donate, fuse=fuse, keep_inputs=keep_inputs).run()


def analyze_subgraph(graph: IRGraph, compute_dtype: str | None = None) -> list:
    """Reference-compatible entry point: the ordered step list."""
    return analyze(graph, compute_dtype).steps
