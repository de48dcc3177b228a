"""Offline compiler tests (no GPU, no native library): op tables, pattern fusion,
lowering, arena planning.  Structure follows the reference's
tests/test_cuda_compiler.py; assertions about NVRTC source text do not apply
because no source is generated."""

import model_zoo as mz
import torch
from cuda_compiler import compile_subgraph, get_cuda_supported_ops, is_cuda_op_supported
from cuda_compiler.cuda_codegen import generate_fused_kernel, is_fusible_elementwise
from cuda_compiler.cuda_program import AliasStep, CUBLASStep, CUDAProgram, FusedKernelStep, ReductionKernelStep, SpecialKernelStep
from cuda_compiler.op_classify import OpCategory, classify_op
from cuda_compiler.subgraph_analyzer import analyze_subgraph
from helpers import graph, masked_softmax_graph, node, rmsnorm_graph, rope_graph, silu_mul_graph, ts
from ir_export import extract_ir
from npu_compiler import load_ir_from_dict

REFERENCE_SUPPORTED = [
    "aten.conv2d.default", "aten.relu.default", "aten.relu_.default", "aten.batch_norm.default", "aten.max_pool2d.default",
    "aten.adaptive_avg_pool2d.default", "aten.linear.default", "aten.matmul.default", "aten.addmm.default", "aten.t.default",
    "aten.add.Tensor", "aten.add_.Tensor", "aten.mul.Tensor", "aten.div.Tensor", "aten.silu.default", "aten.neg.default",
    "aten.rsqrt.default", "aten.cos.default", "aten.sin.default", "aten.pow.Tensor_Scalar", "aten.embedding.default",
    "aten.transpose.int", "aten.cat.default", "aten.slice.Tensor", "aten.expand.default", "aten.index_copy.default",
    "aten.softmax.int", "aten.mean.dim", "aten.full.default", "aten.reshape.default", "aten.view.default",
    "aten.flatten.using_ints", "aten.contiguous.default", "aten.unsqueeze.default", "aten.alias.default", "aten.detach_.default",
    "aten.to.dtype", "aten.dropout.default", "<built-in function getitem>", "aten._assert_tensor_metadata.default",
    "wrap_with_set_grad_enabled",
]


def steps_of(ir, kind):
    return [s for s in analyze_subgraph(load_ir_from_dict(ir)) if isinstance(s, kind)]


def test_classification_matches_reference_table():
    assert classify_op("aten.matmul.default") == OpCategory.ANCHOR_BLAS
    assert classify_op("aten.linear.default") == OpCategory.ANCHOR_BLAS
    assert classify_op("aten.conv2d.default") == OpCategory.ANCHOR_BLAS
    for op in ("aten.relu.default", "aten.silu.default", "aten.add.Tensor", "aten.mul.Tensor"):
        assert classify_op(op) == OpCategory.ELEMENTWISE
    assert classify_op("aten.softmax.int") == OpCategory.REDUCTION
    assert classify_op("aten.reshape.default") == OpCategory.SHAPE_ALIAS
    assert classify_op("aten.view.default") == OpCategory.SHAPE_ALIAS
    assert classify_op("aten.embedding.default") == OpCategory.SPECIAL
    assert classify_op("aten._assert_tensor_metadata.default") == OpCategory.NOOP
    assert classify_op("aten.never_heard_of.default") == OpCategory.SPECIAL


def test_support_set_covers_the_reference_set():
    ops = get_cuda_supported_ops()
    assert all(op in ops for op in REFERENCE_SUPPORTED) and len(ops) >= 30
    assert is_cuda_op_supported("aten.conv2d.default") and is_cuda_op_supported("aten.silu.default", {})
    assert not is_cuda_op_supported("aten.some_weird_op.default")


def test_single_relu_is_one_fused_step():
    ir = graph([node("relu", "aten.relu.default", [ts("x", [1, 256])], [ts("y", [1, 256])])], [ts("x", [1, 256])], [ts("y", [1, 256])])
    fused = steps_of(ir, FusedKernelStep)
    assert len(fused) == 1 and fused[0].total_elements == 256


def test_silu_mul_fuses():
    fused = steps_of(silu_mul_graph(1, 256, "float32"), FusedKernelStep)
    assert len(fused) == 1 and "silu" in fused[0].kernel_name
    assert [op[0] for op in fused[0].params["program"]] == ["SILU", "MUL"]


def test_linear_breaks_chains_and_absorbs_following_relu():
    n = [node("relu1", "aten.relu.default", [ts("x", [1, 256])], [ts("r", [1, 256])]),
         node("linear", "aten.linear.default", [ts("r", [1, 256]), ts("w", [128, 256])], [ts("l", [1, 128])]),
         node("relu2", "aten.relu.default", [ts("l", [1, 128])], [ts("y", [1, 128])])]
    ir = graph(n, [ts("x", [1, 256])], [ts("y", [1, 128])], [ts("w", [128, 256])])
    blas, fused = steps_of(ir, CUBLASStep), steps_of(ir, FusedKernelStep)
    assert len(blas) == 1 and blas[0].params["relu"]       # the reference leaves relu2 as a second fused kernel
    assert len(fused) == 1


def test_multi_consumer_is_a_fusion_barrier():
    n = [node("relu", "aten.relu.default", [ts("x", [1, 256])], [ts("r", [1, 256])]),
         node("add", "aten.add.Tensor", [ts("r", [1, 256]), ts("r", [1, 256])], [ts("y", [1, 256])])]
    assert len(steps_of(graph(n, [ts("x", [1, 256])], [ts("y", [1, 256])]), FusedKernelStep)) == 2


def test_reshape_is_alias():
    ir = graph([node("reshape", "aten.reshape.default", [ts("x", [2, 128])], [ts("y", [256])], shape=[256])], [ts("x", [2, 128])], [ts("y", [256])])
    assert len(steps_of(ir, AliasStep)) == 1 and len(analyze_subgraph(load_ir_from_dict(ir))) == 1


def test_softmax_and_embedding_steps():
    ir = graph([node("softmax", "aten.softmax.int", [ts("x", [4, 128])], [ts("y", [4, 128])], dim=-1)], [ts("x", [4, 128])], [ts("y", [4, 128])])
    red = steps_of(ir, ReductionKernelStep)
    assert len(red) == 1 and red[0].kernel_name == "softmax_kernel" and red[0].params["rows"] == 4
    ir = graph([node("embed", "aten.embedding.default", [ts("weight", [1000, 256]), ts("indices", [4], "int64")], [ts("y", [4, 256])])],
               [ts("indices", [4], "int64")], [ts("y", [4, 256])], [ts("weight", [1000, 256])])
    sp = steps_of(ir, SpecialKernelStep)
    assert len(sp) == 1 and sp[0].kernel_name == "embedding_kernel" and sp[0].params["embed_dim"] == 256


def test_conv_step_and_weight_prep():
    ir = graph([node("conv", "aten.conv2d.default", [ts("x", [1, 8, 8, 8]), ts("w", [16, 8, 3, 3])], [ts("y", [1, 16, 6, 6])],
                     stride=[1, 1], padding=[0, 0], groups=1)], [ts("x", [1, 8, 8, 8])], [ts("y", [1, 16, 6, 6])], [ts("w", [16, 8, 3, 3])])
    prog = compile_subgraph(ir)
    blas = [s for s in prog.steps if isinstance(s, CUBLASStep)]
    assert len(blas) == 1 and blas[0].blas_type == "conv2d" and blas[0].params["out_h"] == 6
    assert len(prog.weight_preps) == 1 and prog.weight_preps[0].kind == "conv_fold"
    # channels-last output: NCHW shape, C has stride 1
    assert prog.views["y"].strides[1] == 1


def test_rmsnorm_chain_becomes_one_kernel():
    for dtype in ("float32", "bfloat16"):
        steps = analyze_subgraph(load_ir_from_dict(rmsnorm_graph(3, 256, dtype)))
        rms = [s for s in steps if isinstance(s, ReductionKernelStep) and s.kernel_name == "rmsnorm_kernel"]
        assert len(rms) == 1 and rms[0].params["cols"] == 256 and abs(rms[0].params["eps"] - 1e-6) < 1e-12
        assert not [s for s in steps if isinstance(s, FusedKernelStep)]


def test_masked_softmax_fusion_with_broadcast_mask():
    red = steps_of(masked_softmax_graph(12, 128), ReductionKernelStep)
    assert len(red) == 1 and red[0].kernel_name == "masked_softmax_kernel"
    assert red[0].params["rows"] == 12 * 128 and red[0].params["cols"] == 128
    assert red[0].params["mask_strides"][1:] == (0, 128)  # head axis broadcast, one row per query


def test_rope_chain_becomes_table_plus_rotate():
    steps = analyze_subgraph(load_ir_from_dict(rope_graph(12, 16)))
    names = [s.kernel_name for s in steps if isinstance(s, SpecialKernelStep)]
    assert names == ["rope_kernel", "rope_rotate_kernel"] and not [s for s in steps if isinstance(s, FusedKernelStep)]


def test_codegen_helpers_keep_reference_names():
    assert is_fusible_elementwise("aten.relu.default") and is_fusible_elementwise("aten.add.Tensor")
    assert not is_fusible_elementwise("aten.matmul.default")
    g = load_ir_from_dict(silu_mul_graph(1, 8, "float32"))
    text = generate_fused_kernel("fused_silu_mul", g.nodes, ["gate", "up"], "y")
    assert "fused_silu_mul" in text and "exp" in text and "*" in text


def test_buffer_plan_reuses_memory():
    prog = compile_subgraph(extract_ir(mz.resnet(18, device="meta"), (torch.zeros(1, 3, 64, 64, device="meta"),), "r18"))
    assert isinstance(prog, CUDAProgram)
    total = sum(a.size_bytes for a in prog.buffer_allocations)
    assert 0 < prog.arena_bytes < total
    live = [a for a in prog.buffer_allocations if a.size_bytes and a.offset >= 0]
    for i, a in enumerate(live):
        for b in live[i + 1:]:
            overlap_mem = a.offset < b.offset + b.size_bytes and b.offset < a.offset + a.size_bytes
            overlap_time = not (a.last_step < b.first_step or b.last_step < a.first_step)
            assert not (overlap_mem and overlap_time), (a, b)


def test_resnet_block_compiles_to_two_convs_with_fused_epilogues():
    prog = compile_subgraph(extract_ir(mz.resnet(18, device="meta"), (torch.zeros(1, 3, 64, 64, device="meta"),), "r18"))
    convs = [s for s in prog.steps if isinstance(s, CUBLASStep) and s.blas_type == "conv2d"]
    assert len(convs) == 20 and all(c.params["bn_folded"] for c in convs)
    assert sum(1 for c in convs if c.params["residual"] is not None) == 8
    assert not [s for s in prog.steps if isinstance(s, ReductionKernelStep) and s.kernel_name == "batch_norm_kernel"]
    assert prog.compute_dtype == "float16"


def test_qwen_mlp_pattern_at_real_sizes():
    x, f32 = ts("x", [1, 1536]), "float32"
    n = [node("gate", "aten.linear.default", [x, ts("gate_w", [8960, 1536])], [ts("g", [1, 8960])]),
         node("up", "aten.linear.default", [x, ts("up_w", [8960, 1536])], [ts("u", [1, 8960])]),
         node("silu", "aten.silu.default", [ts("g", [1, 8960])], [ts("s", [1, 8960])]),
         node("mul", "aten.mul.Tensor", [ts("s", [1, 8960]), ts("u", [1, 8960])], [ts("m", [1, 8960])]),
         node("down", "aten.linear.default", [ts("m", [1, 8960]), ts("down_w", [1536, 8960])], [ts("y", [1, 1536])])]
    ir = graph(n, [x], [ts("y", [1, 1536])], [ts("gate_w", [8960, 1536]), ts("up_w", [8960, 1536]), ts("down_w", [1536, 8960])])
    prog = compile_subgraph(ir)
    blas = [s for s in prog.steps if isinstance(s, CUBLASStep)]
    # gate and up share one GEMM over interleaved rows with the silu*up epilogue; down is the second
    assert len(blas) == 2 and blas[0].params["glu"] and blas[0].params["N"] == 2 * 8960 and blas[1].params["K"] == 8960
    assert [p.kind for p in prog.weight_preps] == ["interleave_rows"]
    assert not [s for s in prog.steps if isinstance(s, FusedKernelStep)]


def _two_rope_graph(T=16, D=128, dtype="bfloat16", reader_between=False):
    """rope(q [1,12,T,D]) and rope(k [1,2,T,D]) over the same cos / sin tables; with ``reader_between`` a neg of
    the rotated q sits before the k chain in node order."""
    inv, pos = ts("inv_freq", [D // 2], "float32"), ts("position_ids", [1, T], "int64")
    cs = lambda n: ts(n, [1, T, D], dtype)
    u = lambda n: ts(n, [1, 1, T, D], dtype)
    n = [node("hop", "wrap_with_set_grad_enabled", [inv, pos], [cs("hop_0"), cs("hop_1")]),
         node("cos", "<built-in function getitem>", [cs("hop_0"), cs("hop_1")], [cs("cos")], index=0),
         node("sin", "<built-in function getitem>", [cs("hop_0"), cs("hop_1")], [cs("sin")], index=1),
         node("cos_u", "aten.unsqueeze.default", [cs("cos")], [u("cos_u")], dim=1),
         node("sin_u", "aten.unsqueeze.default", [cs("sin")], [u("sin_u")], dim=1)]
    outs = []
    for tag, H in (("q", 12), ("k", 2)):
        x = ts(tag, [1, H, T, D], dtype)
        h = lambda nm: ts(f"{tag}_{nm}", [1, H, T, D // 2], dtype)
        f = lambda nm: ts(f"{tag}_{nm}", [1, H, T, D], dtype)
        n += [node(f"{tag}_mul_c", "aten.mul.Tensor", [x, u("cos_u")], [f("mul_c")]),
              node(f"{tag}_lo", "aten.slice.Tensor", [x], [h("lo")], dim=3, start=0, end=D // 2),
              node(f"{tag}_hi", "aten.slice.Tensor", [x], [h("hi")], dim=3, start=D // 2, end=9223372036854775807),
              node(f"{tag}_neg", "aten.neg.default", [h("hi")], [h("neg")]),
              node(f"{tag}_cat", "aten.cat.default", [h("neg"), h("lo")], [f("cat")], dim=-1),
              node(f"{tag}_mul_s", "aten.mul.Tensor", [f("cat"), u("sin_u")], [f("mul_s")]),
              node(f"{tag}_y", "aten.add.Tensor", [f("mul_c"), f("mul_s")], [f("y")])]
        outs.append(f("y"))
        if tag == "q" and reader_between:
            n.append(node("q_after", "aten.neg.default", [f("y")], [f("after")]))
            outs.append(f("after"))
    return graph(n, [ts("q", [1, 12, T, D], dtype), ts("k", [1, 2, T, D], dtype), pos], outs, [inv])


def test_two_ropes_over_the_same_tables_share_a_launch():
    kinds = [getattr(s, "kernel_name", None) for s in analyze_subgraph(load_ir_from_dict(_two_rope_graph()))]
    assert kinds.count("rope_rotate_pair_kernel") == 1 and kinds.count("rope_rotate_kernel") == 0
    # a reader of the first result that comes before the second rotation keeps the two apart (the pair runs where
    # the later rotation was, which would be after that reader)
    kinds = [getattr(s, "kernel_name", None) for s in analyze_subgraph(load_ir_from_dict(_two_rope_graph(reader_between=True)))]
    assert kinds.count("rope_rotate_pair_kernel") == 0 and kinds.count("rope_rotate_kernel") == 2


def test_qwen_prefill_layer_plan():
    L = 2
    cfg = mz.qwen2_config(num_layers=L)
    ir = extract_ir(mz.QwenPrefillWrapper(mz.qwen2_model(cfg)), mz.qwen2_example_inputs(cfg, 1, 128, None), "qp")   # 128 rows: past the decode shapes, whose norms fold into the GEMMs
    prog = compile_subgraph(ir)
    kinds = [getattr(s, "kernel_name", None) or s.blas_type for s in prog.steps if not isinstance(s, AliasStep)]
    # a prefill layer: norm, q/k/v, rope on q and k in one launch, attention, o_proj, norm, gate/up, down
    assert kinds.count("rope_rotate_pair_kernel") == L and kinds.count("rope_rotate_kernel") == 0
    assert kinds.count("attention") == L and kinds.count("rmsnorm_kernel") == 2 * L + 1 and kinds.count("gemm") == 4 * L + 1
    assert (len(kinds) - 4) / L == 8                           # minus embedding, rope table, last norm, lm_head
    pair = next(s for s in prog.steps if getattr(s, "kernel_name", None) == "rope_rotate_pair_kernel")
    assert list(pair.output_buffer_names) == [pair.params["q_out"].buffer, pair.params["k_out"].buffer]
    assert pair.params["q"].buffer == pair.params["k"].buffer   # both are slices of the merged projection's output
    kinds0 = [getattr(s, "kernel_name", None) or s.blas_type for s in compile_subgraph(ir, fuse=False).steps if not isinstance(s, AliasStep)]
    assert "rope_rotate_pair_kernel" not in kinds0
    # 512 tokens: the down projection (12 tiles of 256 x 256, K = 8960) is split over CTA pairs, and the kernel that adds up
    # its partial sums also applies the RMSNorm that follows (the next layer's input norm, the final norm)
    ir512 = extract_ir(mz.QwenPrefillWrapper(mz.qwen2_model(cfg)), mz.qwen2_example_inputs(cfg, 1, 512, None), "qp512")
    prog512 = compile_subgraph(ir512)
    kinds512 = [getattr(s, "kernel_name", None) or s.blas_type for s in prog512.steps if not isinstance(s, AliasStep)]
    tails = [s for s in prog512.steps if isinstance(s, SpecialKernelStep) and s.params.get("norm_tail")]
    assert len(tails) == L and all(t.params["K"] == cfg.intermediate_size and t.params["residual"] is not None for t in tails)
    assert all(t.kernel_name == "gemm_pair_kernel" and len(t.output_buffer_names) == 2 and t.params["op"] == "linear" for t in tails)
    assert kinds512.count("rmsnorm_kernel") == L + 1 and kinds512.count("gemm") == 3 * L + 1


def _assert_arena_is_consistent(prog):
    """Every tensor a step touches lives in a buffer whose live range covers that step (the peepholes move and merge
    steps after lowering), and no two such buffers that are live at the same step share a byte of the arena.
    (Buffers that no step touches any more - the output of a folded RMSNorm - keep a placeholder offset.)"""
    by_name = {a.name: a for a in prog.buffer_allocations}
    used: dict[str, object] = {}
    for i, st in enumerate(prog.steps):
        p = getattr(st, "params", None) or {}
        views = [v for v in p.values() if hasattr(v, "buffer")] + [v for d in p.values() if isinstance(d, dict) for v in d.values() if hasattr(v, "buffer")]
        for v in views:
            a = by_name.get(v.buffer)
            if a is None or a.size_bytes == 0:
                continue
            used[a.name] = a
            if not a.persistent:
                assert a.first_step <= i <= a.last_step, (i, type(st).__name__, p.get("op"), v.buffer, a.first_step, a.last_step)
    # every arena buffer a step reads has been written by an earlier step (donated inputs and persistent buffers aside)
    produced: set[str] = set()
    for i, st in enumerate(prog.steps):
        if isinstance(st, AliasStep):
            continue
        outs = list(getattr(st, "output_buffer_names", None) or [st.output_buffer_name])
        out_bufs = {prog.views[n].buffer if n in prog.views else n for n in outs}
        for n in st.input_buffer_names:
            b = prog.views[n].buffer if n in prog.views else n
            a = by_name.get(b)
            if a is None or a.persistent or a.size_bytes == 0 or b in out_bufs:
                continue
            assert b in produced, (i, getattr(st, "kernel_name", None) or st.blas_type, n, b)
        produced |= out_bufs
    placed = list(used.values())
    assert placed
    for i, a in enumerate(placed):
        assert a.offset % 256 == 0 and a.offset + a.size_bytes <= prog.arena_bytes, a.name
        for b in placed[i + 1:]:
            if a.last_step < b.first_step or b.last_step < a.first_step:
                continue
            assert a.offset + a.size_bytes <= b.offset or b.offset + b.size_bytes <= a.offset, (a.name, b.name)


def test_arena_plans_stay_consistent_after_the_peepholes():
    L = 2
    cfg = mz.qwen2_config(num_layers=L)
    for T in (128, 512):
        ir = extract_ir(mz.QwenPrefillWrapper(mz.qwen2_model(cfg)), mz.qwen2_example_inputs(cfg, 1, T, None), f"qp{T}")
        _assert_arena_is_consistent(compile_subgraph(ir))
    ird = extract_ir(mz.QwenDecodeWrapper(mz.qwen2_model(cfg), L), mz.qwen2_example_inputs(cfg, 2, 1, 256), "qd")
    _assert_arena_is_consistent(compile_subgraph(ird))
    _assert_arena_is_consistent(compile_subgraph(ird, fuse=False))
    _assert_arena_is_consistent(compile_subgraph(extract_ir(mz.resnet(18, device="meta"), (torch.zeros(1, 3, 64, 64, device="meta"),), "r18")))


def test_qwen_decode_layer_plan():
    L = 2
    cfg = mz.qwen2_config(num_layers=L)
    ir = extract_ir(mz.QwenDecodeWrapper(mz.qwen2_model(cfg), L), mz.qwen2_example_inputs(cfg, 2, 1, 256), "qd")
    prog = compile_subgraph(ir)
    assert prog.compute_dtype == "bfloat16"
    kinds = [getattr(s, "kernel_name", None) or s.blas_type for s in prog.steps if not isinstance(s, AliasStep)]
    # decode shapes: every RMSNorm that sits between two GEMMs is folded into them (the producing GEMM
    # writes sum-of-squares partials, the consuming one scales its rows); the first one, fed by the
    # embedding, and the last one, in front of the vocabulary projection (which runs on the persistent
    # kernel), keep their kernels
    assert kinds.count("attention") == L and kinds.count("rmsnorm_kernel") == 2
    # the q/k/v projection of every layer also rotates q and k and writes the new cache rows (its step replaces the rope / cache step)
    fused_qkv = [s.params for s in prog.steps if isinstance(s, SpecialKernelStep) and s.params.get("op") == "linear_qkv_rope"]
    assert len(fused_qkv) == L and all(f["Hq"] == cfg.num_attention_heads and f["Hkv"] == cfg.num_key_value_heads for f in fused_qkv)
    assert kinds.count("gemm") == 3 * L + 1                    # o_proj, gate+up, down (+ lm_head)
    gemms = [s.params for s in prog.steps if isinstance(s, CUBLASStep)] + fused_qkv
    assert sum(1 for g in gemms if g.get("norm")) == 2 * L - 1 and sum(1 for g in gemms if g.get("sumsq_out") is not None) == 2 * L - 1
    assert sorted(p.kind for p in prog.weight_preps).count("scale_cols") == 0          # (the tied head stays as it is)
    assert sum(1 for p in prog.weight_preps if p.params.get("col_scale")) == 2 * L - 1  # q/k/v of layers 1.., gate/up of all
    assert kinds.count("qkv_rope_cache_kernel") == 0 and kinds.count("index_copy_kernel") == 0 and kinds.count("rope_rotate_kernel") == 0
    assert len(prog.donated_inputs) == 2 * L
    per_layer = (len(kinds) - 5) / L                           # minus embedding, rope table, first and last norm, lm_head
    assert per_layer == 5                                      # q/k/v + rope + cache, attention, o_proj, gate/up, down
    # fuse=False keeps every op on its own kernel, with the reference's rounding points
    kinds0 = [getattr(s, "kernel_name", None) or s.blas_type for s in compile_subgraph(ir, fuse=False).steps if not isinstance(s, AliasStep)]
    assert "rmsnorm_kernel" not in kinds0 and kinds0.count("gemm") == 7 * L + 1
    # without donation the cache is copied, as in the reference
    prog2 = compile_subgraph(ir, donate_inputs=False)
    assert not prog2.donated_inputs
    kinds2 = [getattr(s, "kernel_name", None) or s.blas_type for s in prog2.steps if not isinstance(s, AliasStep)]
    assert kinds2.count("index_copy_kernel") == 2 * L and kinds2.count("rope_rotate_kernel") == 2 * L
