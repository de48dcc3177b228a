"""Sub-graph pattern matching: IR node groups -> one fused library call.

The reference fuses three patterns before its generic pass - GQA decode matmuls,
the six-op RMSNorm chain and add+softmax (cuda_compiler/subgraph_analyzer.py:85-160,
667-789) - and then chains same-shape elementwise ops.  This module covers the same
ground and goes further, because on this backend a launch and an HBM round trip are
what a decode step is made of:

* ``b200.rmsnorm``     cast/pow/mean/add/rsqrt/mul/cast/mul            -> one kernel
* ``b200.rope_rotate`` mul/slice/slice/neg/cat/mul/add                 -> one kernel
* ``b200.rope_pair``   rope(q) + rope(k) of a prefill layer                  -> one launch
* ``b200.attention``   repeat_kv + QK^T + scale + mask + softmax + PV + transpose/reshape
* ``b200.softmax``     [scale] + mask add + softmax [+ cast]
* ``b200.linear``      linear + {residual add, relu, silu*up} epilogues
* ``b200.conv2d``      conv + batch-norm folding + {relu, residual add + relu} epilogues

A match replaces its nodes by one synthetic ``OpNode`` placed where the last matched
node stood.  A match is only accepted when every tensor it swallows is invisible
outside (no other consumer, not a graph output), so dropping the intermediate
results is safe.
"""

from __future__ import annotations

from dataclasses import dataclass, field

from npu_compiler.ir_reader import IRGraph, OpNode, TensorSpec

NOOP_OPS = {"aten._assert_tensor_metadata.default"}
# single-input ops whose output is the same values (possibly another dtype)
PASSTHROUGH_OPS = {"aten.dropout.default", "aten.alias.default", "aten.detach_.default", "aten.detach.default",
                   "aten.contiguous.default", "aten.clone.default"}
ADD_OPS = {"aten.add.Tensor", "aten.add_.Tensor"}
MUL_OPS = {"aten.mul.Tensor", "aten.mul_.Tensor"}
RELU_OPS = {"aten.relu.default", "aten.relu_.default"}
SILU_OPS = {"aten.silu.default", "aten.silu_.default"}
RESHAPE_OPS = {"aten.reshape.default", "aten.view.default", "aten._unsafe_view.default"}


@dataclass
class GraphIndex:
    """Producer / consumer maps over a node list."""

    nodes: list[OpNode]
    graph_outputs: set[str]
    position: dict[int, int] = field(default_factory=dict)       # id(node) -> index
    producer: dict[str, OpNode] = field(default_factory=dict)     # tensor -> node
    consumers: dict[str, list[OpNode]] = field(default_factory=dict)
    specs: dict[str, TensorSpec] = field(default_factory=dict)
    taken: set[int] = field(default_factory=set)                  # ids of nodes an earlier match owns

    @classmethod
    def build(cls, nodes: list[OpNode], graph: IRGraph) -> "GraphIndex":
        gi = cls(nodes=nodes, graph_outputs={o.name for o in graph.graph_outputs})
        for spec in list(graph.graph_inputs) + list(graph.weights):
            gi.specs[spec.name] = spec
        for placeholder, key in graph.weight_name_mapping.items():
            for w in graph.weights:
                if w.name == key:
                    gi.specs.setdefault(placeholder, TensorSpec(placeholder, w.shape, w.dtype))
        for i, n in enumerate(nodes):
            gi.position[id(n)] = i
            for t in n.inputs:
                gi.consumers.setdefault(t.name, []).append(n)
                gi.specs.setdefault(t.name, t)
            for t in n.outputs:
                gi.producer[t.name] = n
                gi.specs[t.name] = t
        return gi

    def prod(self, name: str, *ops: str) -> OpNode | None:
        n = self.producer.get(name)
        if n is None or (ops and n.op_type not in ops):
            return None
        return n

    def sole_consumer(self, name: str, *ops: str) -> OpNode | None:
        if name in self.graph_outputs:
            return None
        cs = self.consumers.get(name, [])
        if len(cs) != 1 or (ops and cs[0].op_type not in ops) or id(cs[0]) in self.taken:
            return None
        return cs[0]

    def shape(self, name: str) -> list[int]:
        return list(self.specs[name].shape)


def _scalar(node: OpNode, key: str = "other"):
    v = node.attrs.get(key)
    return v if isinstance(v, (int, float)) and not isinstance(v, bool) else None


def _other_input(node: OpNode, name: str) -> TensorSpec | None:
    if len(node.inputs) != 2:
        return None
    a, b = node.inputs
    if a.name == name and b.name != name:
        return b
    if b.name == name and a.name != name:
        return a
    return None


def _norm_dim(d: int, ndim: int) -> int:
    return d + ndim if d < 0 else d


def _macro(op: str, last: OpNode, inputs: list[TensorSpec], outputs: list[TensorSpec], attrs: dict, matched: list[OpNode]) -> OpNode:
    node = OpNode(name=f"{op.split('.')[-1]}__{last.name}", op_type=op, inputs=inputs, outputs=outputs, attrs=dict(attrs))
    node.attrs["_orig"] = matched
    return node


# ---------------------------------------------------------------------------
# individual patterns: each returns (matched_nodes, macro_node) or None
# ---------------------------------------------------------------------------
def match_rmsnorm(gi: GraphIndex, pow_node: OpNode):
    """``x -> [to f32] -> pow 2 -> mean(-1) -> +eps -> rsqrt -> * x -> [to act] -> * w``
    (reference matcher: subgraph_analyzer.py:667-756)."""
    if pow_node.op_type != "aten.pow.Tensor_Scalar" or pow_node.attrs.get("exponent") not in (2, 2.0):
        return None
    x32 = pow_node.inputs[0]
    ndim = len(x32.shape)
    mean = gi.sole_consumer(pow_node.outputs[0].name, "aten.mean.dim")
    if mean is None:
        return None
    dims = mean.attrs.get("dim", [-1])
    dims = [dims] if isinstance(dims, int) else list(dims)
    if [_norm_dim(d, ndim) for d in dims] != [ndim - 1] or mean.outputs[0].shape[-1:] != [1]:
        return None
    add = gi.sole_consumer(mean.outputs[0].name, *ADD_OPS)
    if add is None or _scalar(add) is None:
        return None
    rsqrt = gi.sole_consumer(add.outputs[0].name, "aten.rsqrt.default")
    if rsqrt is None:
        return None
    mul1 = gi.sole_consumer(rsqrt.outputs[0].name, *MUL_OPS)
    if mul1 is None:
        return None
    other = _other_input(mul1, rsqrt.outputs[0].name)
    if other is None or other.name != x32.name:
        return None
    matched = [pow_node, mean, add, rsqrt, mul1]
    cur, round_mid = mul1.outputs[0], False
    cast = gi.sole_consumer(cur.name, "aten.to.dtype")
    if cast is not None:
        matched.append(cast)
        round_mid = cast.outputs[0].dtype != cur.dtype
        cur = cast.outputs[0]
    mul2 = gi.sole_consumer(cur.name, *MUL_OPS)
    if mul2 is None:
        return None
    w = _other_input(mul2, cur.name)
    if w is None or list(w.shape) != [x32.shape[-1]]:
        return None
    matched.append(mul2)
    x = x32
    up = gi.prod(x32.name, "aten.to.dtype")
    if up is not None and all(c in (pow_node, mul1) for c in gi.consumers.get(x32.name, [])) and x32.name not in gi.graph_outputs:
        matched.insert(0, up)
        x = up.inputs[0]
    attrs = {"eps": float(_scalar(add)), "round_mid": bool(round_mid)}
    return matched, _macro("b200.rmsnorm", mul2, [x, w], [mul2.outputs[0]], attrs, matched)


def match_rope_rotate(gi: GraphIndex, add: OpNode):
    """``x*cos + cat(-x[..., D/2:], x[..., :D/2]) * sin`` (rotate_half form)."""
    if add.op_type not in ADD_OPS or len(add.inputs) != 2:
        return None
    muls = [gi.prod(t.name, *MUL_OPS) for t in add.inputs]
    if None in muls or muls[0] is muls[1]:
        return None
    for mul_x, mul_r in (muls, muls[::-1]):
        if len(mul_x.inputs) != 2 or len(mul_r.inputs) != 2:
            continue
        cat = None
        for t in mul_r.inputs:
            c = gi.prod(t.name, "aten.cat.default")
            if c is not None:
                cat, sin_u = c, _other_input(mul_r, t.name)
        if cat is None or sin_u is None or len(cat.inputs) != 2:
            continue
        nd = len(cat.outputs[0].shape)
        D = cat.outputs[0].shape[-1]
        if _norm_dim(cat.attrs.get("dim", 0), nd) != nd - 1 or nd != 4 or D % 16:
            continue
        neg = gi.prod(cat.inputs[0].name, "aten.neg.default")
        s_lo = gi.prod(cat.inputs[1].name, "aten.slice.Tensor")
        s_hi = gi.prod(neg.inputs[0].name, "aten.slice.Tensor") if neg is not None else None
        if neg is None or s_lo is None or s_hi is None:
            continue
        x = s_lo.inputs[0]
        if s_hi.inputs[0].name != x.name or list(x.shape) != list(cat.outputs[0].shape):
            continue

        def rng(s):
            return (_norm_dim(s.attrs.get("dim", 0), nd), s.attrs.get("start", 0) or 0, s.attrs.get("end"), s.attrs.get("step", 1) or 1)

        if rng(s_lo)[:2] != (nd - 1, 0) or rng(s_lo)[2] != D // 2 or rng(s_lo)[3] != 1:
            continue
        hi = rng(s_hi)
        if hi[0] != nd - 1 or hi[1] != D // 2 or not (hi[2] is None or hi[2] >= D) or hi[3] != 1:
            continue
        cos_u = _other_input(mul_x, x.name)
        if cos_u is None:
            continue
        B, H, T, _ = x.shape
        if list(cos_u.shape) != [B, 1, T, D] or list(sin_u.shape) != [B, 1, T, D]:
            continue
        matched = [s_lo, s_hi, neg, cat, mul_x, mul_r, add]
        matched.sort(key=lambda n: gi.position[id(n)])
        return matched, _macro("b200.rope_rotate", add, [x, cos_u, sin_u], [add.outputs[0]], {}, matched)
    return None


def _strip_repeat_kv(gi: GraphIndex, t: TensorSpec, matched: list[OpNode]) -> TensorSpec | None:
    """``reshape(expand(unsqueeze(kv, 2), [B,Hkv,G,S,D]), [B,Hq,S,D])`` -> kv."""
    r = gi.prod(t.name, *RESHAPE_OPS)
    if r is None:
        return t
    e = gi.prod(r.inputs[0].name, "aten.expand.default")
    u = gi.prod(e.inputs[0].name, "aten.unsqueeze.default") if e is not None else None
    if e is None or u is None or u.attrs.get("dim") != 2:
        return None
    kv = u.inputs[0]
    if len(kv.shape) != 4 or len(e.outputs[0].shape) != 5:
        return None
    B, Hkv, S, D = kv.shape
    G = e.outputs[0].shape[2]
    if list(e.outputs[0].shape) != [B, Hkv, G, S, D] or list(r.outputs[0].shape) != [B, Hkv * G, S, D]:
        return None
    matched += [u, e, r]
    return kv


def match_attention(gi: GraphIndex, sm: OpNode):
    """Scaled-dot-product attention with an additive mask and GQA key/value sharing
    (the decode form is what the reference's GQA pre-pass targets,
    subgraph_analyzer.py:85-160 / 819-861)."""
    if sm.op_type not in ("aten.softmax.int", "aten._softmax.default"):
        return None
    nd = len(sm.inputs[0].shape)
    if nd != 4 or _norm_dim(sm.attrs.get("dim", -1), nd) != 3:
        return None
    matched: list[OpNode] = [sm]
    cur = sm.inputs[0]
    mask = None
    add = gi.prod(cur.name, *ADD_OPS)
    if add is not None and len(add.inputs) == 2:
        if gi.sole_consumer(cur.name) is not sm:
            return None
        cand = [t for t in add.inputs if gi.prod(t.name, "aten.matmul.default", *MUL_OPS, "aten.div.Tensor") is not None]
        if len(cand) != 1:
            return None
        cur = cand[0]
        mask = _other_input(add, cur.name)
        if mask is None:
            return None
        matched.append(add)
    scale = 1.0
    sc = gi.prod(cur.name, *MUL_OPS, "aten.div.Tensor")
    if sc is not None and len(sc.inputs) == 1 and _scalar(sc) is not None:
        if len(gi.consumers.get(cur.name, [])) != 1:
            return None
        scale = float(_scalar(sc)) if sc.op_type in MUL_OPS else 1.0 / float(_scalar(sc))
        matched.append(sc)
        cur = sc.inputs[0]
    mm1 = gi.prod(cur.name, "aten.matmul.default")
    if mm1 is None or len(gi.consumers.get(cur.name, [])) != 1:
        return None
    matched.append(mm1)
    q, kT = mm1.inputs
    tr = gi.prod(kT.name, "aten.transpose.int")
    if tr is None or {_norm_dim(tr.attrs.get("dim0"), 4), _norm_dim(tr.attrs.get("dim1"), 4)} != {2, 3}:
        return None
    matched.append(tr)
    k = _strip_repeat_kv(gi, tr.inputs[0], matched)
    if k is None:
        return None
    # forward: softmax -> [cast] -> [dropout] -> matmul(., v)
    cur = sm.outputs[0]
    while True:
        nxt = gi.sole_consumer(cur.name)
        if nxt is None:
            return None
        if nxt.op_type == "aten.to.dtype" or (nxt.op_type in PASSTHROUGH_OPS and
                                                 (nxt.op_type != "aten.dropout.default" or not nxt.attrs.get("train", False)
                                                  or not nxt.attrs.get("p", 0.0))):
            matched.append(nxt)
            cur = nxt.outputs[0]
            continue
        break
    mm2 = nxt
    if mm2.op_type != "aten.matmul.default" or mm2.inputs[0].name != cur.name:
        return None
    matched.append(mm2)
    v = _strip_repeat_kv(gi, mm2.inputs[1], matched)
    if v is None:
        return None
    B, Hq, T, D = q.shape
    if len(k.shape) != 4 or list(k.shape) != list(v.shape) or k.shape[0] != B or k.shape[3] != D or D != 128:
        return None
    Hkv, S = k.shape[1], k.shape[2]
    if Hq % Hkv or (T == 1 and Hq // Hkv > 8):
        return None
    if mask is not None:
        ms = list(mask.shape)
        if len(ms) != 4 or ms[1] != 1 or ms[3] != S or ms[0] not in (1, B) or ms[2] not in (1, T):
            return None
    # tail: transpose(1,2) -> [contiguous] -> reshape [B,T,Hq*D]
    tail = gi.sole_consumer(mm2.outputs[0].name, "aten.transpose.int")
    if tail is None or {_norm_dim(tail.attrs.get("dim0"), 4), _norm_dim(tail.attrs.get("dim1"), 4)} != {1, 2}:
        return None
    matched.append(tail)
    cur = tail.outputs[0]
    nxt = gi.sole_consumer(cur.name)
    if nxt is not None and nxt.op_type in ("aten.contiguous.default", "aten.clone.default"):
        matched.append(nxt)
        cur = nxt.outputs[0]
        nxt = gi.sole_consumer(cur.name)
    if nxt is None or nxt.op_type not in RESHAPE_OPS or list(nxt.outputs[0].shape) != [B, T, Hq * D]:
        return None
    matched.append(nxt)
    matched.sort(key=lambda n: gi.position[id(n)])
    inputs = [q, k, v] + ([mask] if mask is not None else [])
    attrs = {"scale": scale, "has_mask": mask is not None, "B": B, "Hq": Hq, "Hkv": Hkv, "T": T, "S": S, "D": D}
    return matched, _macro("b200.attention", matched[-1], inputs, [nxt.outputs[0]], attrs, matched)


def match_masked_softmax(gi: GraphIndex, sm: OpNode):
    """``[x*scale] + mask -> softmax -> [cast]`` (reference: subgraph_analyzer.py:759-789)."""
    if sm.op_type not in ("aten.softmax.int", "aten._softmax.default"):
        return None
    nd = len(sm.inputs[0].shape)
    if _norm_dim(sm.attrs.get("dim", -1), nd) != nd - 1:
        return None
    add = gi.prod(sm.inputs[0].name, *ADD_OPS)
    if add is None or len(add.inputs) != 2 or gi.sole_consumer(add.outputs[0].name) is not sm:
        return None
    a, b = add.inputs
    out_shape = list(sm.inputs[0].shape)
    if list(a.shape) == out_shape:
        scores, mask = a, b
    elif list(b.shape) == out_shape:
        scores, mask = b, a
    else:
        return None
    matched = [add, sm]
    scale = 1.0
    sc = gi.prod(scores.name, *MUL_OPS)
    if sc is not None and len(sc.inputs) == 1 and _scalar(sc) is not None and gi.sole_consumer(scores.name) is add:
        scale = float(_scalar(sc))
        matched.insert(0, sc)
        scores = sc.inputs[0]
    out = sm.outputs[0]
    cast = gi.sole_consumer(out.name, "aten.to.dtype")
    if cast is not None:
        matched.append(cast)
        out = cast.outputs[0]
    last = matched[-1]
    return matched, _macro("b200.softmax", last, [scores, mask], [out], {"scale": scale, "sum_dtype": add.outputs[0].dtype}, matched)


def match_linear_epilogue(gi: GraphIndex, lin: OpNode):
    """linear -> {+ residual, relu, silu(.) * up}."""
    if lin.op_type != "aten.linear.default" or len(lin.inputs) < 2:
        return None
    out = lin.outputs[0]
    matched = [lin]
    inputs = list(lin.inputs)
    attrs = {"has_bias": len(lin.inputs) > 2, "residual": False, "relu": False, "silu_mul": False, "glu": False}
    nxt = gi.sole_consumer(out.name)
    if nxt is not None and nxt.op_type in ADD_OPS and len(nxt.inputs) == 2 and nxt.attrs.get("alpha", 1) in (1, 1.0):
        res = _other_input(nxt, out.name)
        if res is not None and list(res.shape) == list(out.shape) and res.dtype == out.dtype:
            matched.append(nxt)
            inputs.append(res)
            attrs["residual"] = True
            out = nxt.outputs[0]
            nxt = gi.sole_consumer(out.name)
    if nxt is not None and nxt.op_type in RELU_OPS:
        matched.append(nxt)
        attrs["relu"] = True
        out = nxt.outputs[0]
    elif nxt is not None and nxt.op_type in SILU_OPS and not attrs["residual"]:
        mul = gi.sole_consumer(nxt.outputs[0].name, *MUL_OPS)
        up = _other_input(mul, nxt.outputs[0].name) if mul is not None else None
        if up is not None and list(up.shape) == list(out.shape) and up.dtype == out.dtype:
            matched += [nxt, mul]
            out = mul.outputs[0]
            # gate and up read the same activation: one GEMM over interleaved weights
            upl = gi.prod(up.name, "aten.linear.default")
            if (upl is not None and len(upl.inputs) == 2 and len(lin.inputs) == 2 and upl.inputs[0].name == lin.inputs[0].name
                    and gi.sole_consumer(up.name) is mul and list(upl.inputs[1].shape) == list(lin.inputs[1].shape)
                    and lin.inputs[1].shape[0] % 64 == 0 and gi.prod(lin.inputs[1].name) is None and gi.prod(upl.inputs[1].name) is None):
                matched.insert(0, upl)
                inputs.append(upl.inputs[1])
                attrs["glu"] = True
            else:
                inputs.append(up)
                attrs["silu_mul"] = True
    if len(matched) == 1:
        return None
    matched.sort(key=lambda n: gi.position[id(n)])
    return matched, _macro("b200.linear", matched[-1], inputs, [out], attrs, matched)


def match_conv(gi: GraphIndex, conv: OpNode):
    """conv2d -> [batch_norm (inference)] -> [+ residual] -> [relu]."""
    if conv.op_type != "aten.conv2d.default":
        return None
    matched = [conv]
    inputs = list(conv.inputs)  # x, w, [bias]
    attrs = {k: conv.attrs.get(k) for k in ("stride", "padding", "dilation", "groups")}
    attrs.update(has_bias=len(conv.inputs) > 2, bn=False, residual=False, relu=False, eps=0.0)
    out = conv.outputs[0]
    bn = gi.sole_consumer(out.name, "aten.batch_norm.default")
    if bn is not None and not bn.attrs.get("training", False) and len(bn.inputs) == 5:
        matched.append(bn)
        inputs += bn.inputs[1:]
        attrs.update(bn=True, eps=float(bn.attrs.get("eps", 1e-5)))
        out = bn.outputs[0]
    nxt = gi.sole_consumer(out.name)
    if nxt is not None and nxt.op_type in ADD_OPS and len(nxt.inputs) == 2 and nxt.attrs.get("alpha", 1) in (1, 1.0):
        res = _other_input(nxt, out.name)
        if res is not None and list(res.shape) == list(out.shape):
            matched.append(nxt)
            inputs.append(res)
            attrs["residual"] = True
            out = nxt.outputs[0]
            nxt = gi.sole_consumer(out.name)
    if nxt is not None and nxt.op_type in RELU_OPS:
        matched.append(nxt)
        attrs["relu"] = True
        out = nxt.outputs[0]
    return matched, _macro("b200.conv2d", matched[-1], inputs, [out], attrs, matched)


# ---------------------------------------------------------------------------
# driver
# ---------------------------------------------------------------------------
def _acceptable(gi: GraphIndex, matched: list[OpNode], macro: OpNode) -> bool:
    inside = {id(n) for n in matched}
    keep = {t.name for t in macro.outputs}
    last = max(gi.position[id(n)] for n in matched)
    for n in matched:
        for t in n.outputs:
            outside = [c for c in gi.consumers.get(t.name, []) if id(c) not in inside]
            if t.name in keep:
                if any(gi.position[id(c)] < last for c in outside):
                    return False
            elif outside or t.name in gi.graph_outputs:
                return False
    return True


def apply_patterns(nodes: list[OpNode], graph: IRGraph, families) -> list[OpNode]:
    """Run each pattern family over the node list in order; ``families`` is a list of
    ``(anchor_op_types, matcher)``.  Returns the rewritten node list."""
    for anchor_ops, matcher in families:
        gi = GraphIndex.build(nodes, graph)
        taken = gi.taken
        replace_at: dict[int, OpNode] = {}
        for n in nodes:
            if id(n) in taken or n.op_type not in anchor_ops:
                continue
            m = matcher(gi, n)
            if m is None:
                continue
            matched, macro = m
            if any(id(x) in taken for x in matched) or not _acceptable(gi, matched, macro):
                continue
            taken.update(id(x) for x in matched)
            last = max(matched, key=lambda x: gi.position[id(x)])
            replace_at[id(last)] = macro
        if taken:
            nodes = [replace_at.get(id(n), n) for n in nodes if id(n) not in taken or id(n) in replace_at]
    return nodes


def group_linears(nodes: list[OpNode], graph: IRGraph) -> list[OpNode]:
    """Linears that read the same activation (q/k/v projections) become one GEMM over the
    row-concatenated weights; the member outputs turn into column slices of its result.
    The fused node takes the place of the first member: its operands (the shared input and
    graph-level weights) are all defined there."""
    weight_names = {w.name for w in graph.weights} | set(graph.weight_name_mapping)
    groups: dict[tuple, list[OpNode]] = {}
    for n in nodes:
        if n.op_type != "aten.linear.default" or len(n.inputs) not in (2, 3) or len(n.outputs) != 1:
            continue
        if any(t.name not in weight_names for t in n.inputs[1:]):
            continue
        x, w = n.inputs[0], n.inputs[1]
        key = (x.name, len(n.inputs), w.shape[1], w.dtype, n.outputs[0].dtype, tuple(n.outputs[0].shape[:-1]))
        groups.setdefault(key, []).append(n)
    replace: dict[int, OpNode] = {}
    drop: set[int] = set()
    for members in groups.values():
        if len(members) < 2:
            continue
        first = members[0]
        inputs = [first.inputs[0]]
        for m in members:
            inputs += list(m.inputs[1:])
        macro = OpNode(name=f"linear_group__{first.name}", op_type="b200.linear_group", inputs=inputs,
                       outputs=[m.outputs[0] for m in members],
                       attrs={"has_bias": len(first.inputs) == 3, "n_parts": len(members), "_orig": members})
        replace[id(first)] = macro
        drop.update(id(m) for m in members[1:])
    if not replace:
        return nodes
    return [replace.get(id(n), n) for n in nodes if id(n) not in drop]


def fuse_qkv_post(nodes: list[OpNode], graph: IRGraph) -> list[OpNode]:
    """rope(q), rope(k) -> index_copy into the key cache, v -> index_copy into the value
    cache: one launch.  Runs after the rope pattern, on ``b200.rope_rotate`` nodes."""
    gi = GraphIndex.build(nodes, graph)
    replace: dict[int, OpNode] = {}
    drop: set[int] = set()
    for ic_k in nodes:
        if ic_k.op_type != "aten.index_copy.default" or id(ic_k) in drop or len(ic_k.inputs) != 3:
            continue
        cache_k, index, src = ic_k.inputs
        if len(cache_k.shape) != 4 or _norm_dim(ic_k.attrs.get("dim", 0), 4) != 2:
            continue
        rk = gi.prod(src.name, "b200.rope_rotate")
        if rk is None or gi.sole_consumer(src.name) is not ic_k or id(rk) in drop:
            continue
        k, cos_u, sin_u = rk.inputs
        rq = next((n for n in nodes if n.op_type == "b200.rope_rotate" and n is not rk and id(n) not in drop
                   and n.inputs[1].name == cos_u.name and n.inputs[2].name == sin_u.name
                   and n.inputs[0].shape[0] == k.shape[0] and n.inputs[0].shape[2:] == k.shape[2:]), None)
        if rq is None:
            continue
        ic_v = None
        for n in nodes[gi.position[id(ic_k)] + 1: gi.position[id(ic_k)] + 4]:
            if (n.op_type == "aten.index_copy.default" and len(n.inputs) == 3 and n.inputs[1].name == index.name
                    and list(n.inputs[0].shape) == list(cache_k.shape) and list(n.inputs[2].shape) == list(k.shape)
                    and _norm_dim(n.attrs.get("dim", 0), 4) == 2 and gi.prod(n.inputs[2].name, "b200.rope_rotate") is None):
                ic_v = n
                break
        if ic_v is None or k.shape[2] != index.shape[0]:
            continue
        matched = sorted([rq, rk, ic_k, ic_v], key=lambda n: gi.position[id(n)])
        macro = _macro("b200.qkv_post", matched[-1], [rq.inputs[0], k, ic_v.inputs[2], cos_u, sin_u, cache_k, ic_v.inputs[0], index],
                       [rq.outputs[0], ic_k.outputs[0], ic_v.outputs[0]], {"dim": 2}, matched)
        if not _acceptable(gi, matched, macro):
            continue
        replace[id(matched[-1])] = macro
        drop.update(id(n) for n in matched[:-1])
    if not replace:
        return nodes
    return [replace.get(id(n), n) for n in nodes if id(n) not in drop]



def fuse_rope_pair(nodes: list[OpNode], graph: IRGraph) -> list[OpNode]:
    """rope(q) and rope(k) of one attention layer (same cos / sin tables, batch, positions and
    head dimension) that ``fuse_qkv_post`` left alone - a prefill layer, whose keys go to a
    graph output instead of a cache: one launch for both.  The pair sits where the later of the
    two was."""
    gi = GraphIndex.build(nodes, graph)
    replace: dict[int, OpNode] = {}
    drop: set[int] = set()
    ropes = [n for n in nodes if n.op_type == "b200.rope_rotate"]
    for a in ropes:
        if id(a) in drop or id(a) in replace:
            continue
        xa, cos_u, sin_u = a.inputs
        b = next((n for n in ropes if n is not a and id(n) not in drop and id(n) not in replace
                  and gi.position[id(n)] > gi.position[id(a)]
                  and n.inputs[1].name == cos_u.name and n.inputs[2].name == sin_u.name and n.inputs[0].dtype == xa.dtype
                  and len(n.inputs[0].shape) == 4 and len(xa.shape) == 4
                  and n.inputs[0].shape[0] == xa.shape[0] and list(n.inputs[0].shape[2:]) == list(xa.shape[2:])), None)
        if b is None:
            continue
        matched = [a, b]
        macro = _macro("b200.rope_pair", b, [xa, b.inputs[0], cos_u, sin_u], [a.outputs[0], b.outputs[0]], {}, matched)
        if not _acceptable(gi, matched, macro):
            continue
        replace[id(b)] = macro
        drop.add(id(a))
    if not replace:
        return nodes
    return [replace.get(id(n), n) for n in nodes if id(n) not in drop]


DEFAULT_FAMILIES = [
    ({"aten.pow.Tensor_Scalar"}, match_rmsnorm),
    (ADD_OPS, match_rope_rotate),
    ({"aten.softmax.int", "aten._softmax.default"}, match_attention),
    ({"aten.softmax.int", "aten._softmax.default"}, match_masked_softmax),
    ({"aten.conv2d.default"}, match_conv),
    ({"aten.linear.default"}, match_linear_epilogue),
]
