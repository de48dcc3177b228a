"""Model-level parity on the GPU: IR -> compile_subgraph -> DAGExecutor/CUDABackend ->
kernels, against the CPU oracle on the same seeded inputs, with the tolerances the
reference's own end-to-end tests use (ResNet-18 1e-1 + arg-max, ResNet-50 2e-1 + arg-max:
tests/test_e2e_resnet.py:223-271; Qwen top-5 overlap >= 3 and last-position top-1:
tests/test_e2e_qwen.py:126-137)."""

from pathlib import Path

import numpy as np
import pytest
import torch

import model_zoo as mz
from helpers import np_inputs, run_backend, to_f32
from ir_export import extract_ir
from oracle.ir_interpreter import IRInterpreter, torch_to_numpy

pytestmark = pytest.mark.gpu
GOLDEN = Path(__file__).parent / "golden"


def top5_equal(a, b):
    return (np.sort(np.argsort(-a, -1)[..., :5], -1) == np.sort(np.argsort(-b, -1)[..., :5], -1)).all()


def test_golden_resnet18_fixture():
    fx = np.load(GOLDEN / "resnet18_b2_64.npz")
    m = mz.resnet(18, seed=0)
    ir = extract_ir(m, (torch.from_numpy(fx["x"]),), "resnet18")
    out, _ = run_backend(ir, mz.state_dict_numpy(m.state_dict()), {"x": fx["x"]})
    got = to_f32(out[ir["graph_outputs"][0]["name"]])
    assert np.abs(got - fx["logits"]).max() <= 1e-1 and (got.argmax(-1) == fx["logits"].argmax(-1)).all()


@pytest.mark.parametrize("depth,batch,tol", [(18, 1, 1e-1), (50, 2, 2e-1)])
def test_resnet_vs_fp32_oracle(depth, batch, tol):
    """fp16 on the GPU against the fp32 oracle.  The reference's absolute tolerances
    (1e-1 / 2e-1) were chosen for logits of magnitude ~10; with the seeded random
    initialisation the logits reach several hundred, so the bound scales with them."""
    m = mz.resnet(depth, seed=0)
    x = torch.randn(batch, 3, 224, 224, generator=torch.Generator().manual_seed(0))
    ir = extract_ir(m, (x,), f"resnet{depth}")
    ref = to_f32(list(IRInterpreter(ir, m.state_dict()).execute({"x": x}).values())[0])
    out, dag = run_backend(ir, mz.state_dict_numpy(m.state_dict()), {"x": x.numpy()})
    name = ir["graph_outputs"][0]["name"]
    got = to_f32(out[name])
    assert np.isfinite(got).all()
    bound = tol * max(1.0, float(np.abs(ref).max()) / 10.0)
    assert np.abs(got - ref).max() <= bound, (np.abs(got - ref).max(), bound)
    assert (got.argmax(-1) == ref.argmax(-1)).all() and top5_equal(got, ref)
    # replays (second run captures a CUDA graph, third replays it) agree; the split-K
    # classifier GEMM sums its partials with atomics, so the last bit may differ
    for _ in range(2):
        again = to_f32(dag.execute({"x": x.numpy()})[name].to_numpy())
        np.testing.assert_allclose(again, got, rtol=2e-3, atol=2e-3)


def _qwen(L):
    cfg = mz.qwen2_config(num_layers=L)
    return cfg, mz.qwen2_weights(cfg, seed=0), mz.qwen2_model(cfg)


def test_qwen_prefill_2_layers_full_width():
    L, T = 2, 512
    cfg, sd, model = _qwen(L)
    ir = extract_ir(mz.QwenPrefillWrapper(model), mz.qwen2_example_inputs(cfg, 1, T, None), "qp")
    g = torch.Generator().manual_seed(0)
    ins = (torch.randint(0, cfg.vocab_size, (1, T), generator=g), mz.causal_mask(1, T, T, 0), torch.arange(T)[None], torch.arange(T))
    ref = IRInterpreter(ir, sd).execute(ins)
    out, _ = run_backend(ir, mz.state_dict_numpy(sd), np_inputs(ir, ins))
    names = [o["name"] for o in ir["graph_outputs"]]
    got, want = to_f32(out[names[0]])[0], to_f32(ref[names[0]])[0]
    err = np.abs(got - want).max()
    assert err < 0.15, err
    overlap = [len(set(np.argsort(-got[t])[:5]) & set(np.argsort(-want[t])[:5])) for t in range(T)]
    assert min(overlap) >= 3
    # last position: same top-1 unless the oracle's own top-2 are closer than the logits error
    top2 = np.sort(want[-1])[-2:]
    assert got[-1].argmax() == want[-1].argmax() or top2[1] - top2[0] < 2 * err
    for n in names[1:]:  # K/V caches: rope + projection only, last-bit differences
        a, b = out[n].view(np.uint16).astype(np.int32), ref[n].contiguous().view(torch.uint16).numpy().astype(np.int32)
        assert np.abs(to_f32(out[n]) - to_f32(ref[n])).max() < 0.1
        del a, b


@pytest.mark.parametrize("B", [1, 8])
def test_qwen_decode_greedy_steps_match_oracle(B):
    """A few lock-step greedy decode steps over a 4352-row cache with 4096 rows filled."""
    L, S, P, steps = 2, 4352, 4096, 3
    cfg, sd, model = _qwen(L)
    ir = extract_ir(mz.QwenDecodeWrapper(model, L), mz.qwen2_example_inputs(cfg, B, 1, S), "qd")
    g = torch.Generator().manual_seed(1)
    kv = [(torch.randn(B, 2, S, 128, generator=g) * 0.5).bfloat16() for _ in range(2 * L)]
    ids = torch.randint(0, cfg.vocab_size, (B, 1), generator=g)
    names_in = [s["name"] for s in ir["graph_inputs"]]
    names_out = [o["name"] for o in ir["graph_outputs"]]

    from cuda_compiler import compile_subgraph, is_cuda_op_supported
    from cuda_runtime import CUDABackend, CUDABuffer
    from npu_compiler import partition
    from npu_runtime import DAGExecutor

    dag = DAGExecutor(partition(ir, is_cuda_op_supported), CUDABackend(), compile_subgraph)
    dag.load_weights(mz.state_dict_numpy(sd))
    dev_kv = [CUDABuffer.from_numpy(torch_to_numpy(t)) for t in kv]
    interp = IRInterpreter(ir, sd)
    ref_kv, ref_ids, dev_ids = list(kv), ids.clone(), ids.clone()
    for step in range(steps):
        pos = P + step
        fixed = (mz.causal_mask(B, 1, S, pos), torch.full((B, 1), pos), torch.tensor([pos]))
        ref = interp.execute((ref_ids, *fixed, *ref_kv))
        feed = dict(zip(names_in, [dev_ids.numpy()] + [torch_to_numpy(t) for t in fixed] + dev_kv))
        out = dag.execute(feed)
        got, want = to_f32(out[names_out[0]])[:, 0], to_f32(ref[names_out[0]])[:, 0]
        err = np.abs(got - want).max()
        assert err < 0.15, (step, err)
        for b in range(B):
            top2 = np.sort(want[b])[-2:]
            assert got[b].argmax() == want[b].argmax() or top2[1] - top2[0] < 2 * err
        # the new cache row is written where the oracle writes it; all other rows are untouched (bit-exact)
        k0 = out[names_out[1]].to_numpy()
        want_k0 = torch_to_numpy(ref[names_out[1]])
        untouched = np.ones(S, bool)
        untouched[P:pos + 1] = False   # rows written in this and earlier steps carry floating-point results
        np.testing.assert_array_equal(k0.view(np.uint16)[:, :, untouched], want_k0.view(np.uint16)[:, :, untouched])
        assert np.abs(to_f32(k0[:, :, P:pos + 1]) - to_f32(want_k0[:, :, P:pos + 1])).max() < 0.05
        # feed both sides the oracle's token so that the runs stay comparable; caches stay on the device
        ref_ids = dev_ids = torch.from_numpy(want.argmax(-1))[:, None]
        ref_kv = [ref[n] for n in names_out[1:]]
        dev_kv = [out[n] for n in names_out[1:]]


def test_qwen_tiny_golden_fixture_on_gpu():
    from golden.make_golden import tiny_qwen

    fx = np.load(GOLDEN / "qwen_tiny.npz")
    cfg, sd, model = tiny_qwen()
    T = int(fx["T"])
    ir = extract_ir(mz.QwenPrefillWrapper(model), mz.qwen2_example_inputs(cfg, 1, T, None, device="cpu"), "p")
    ins = np_inputs(ir, (torch.from_numpy(fx["ids"]), mz.causal_mask(1, T, T, 0), torch.arange(T)[None], torch.arange(T)))
    out, _ = run_backend(ir, mz.state_dict_numpy(sd), ins)
    gold = torch.from_numpy(fx["prefill_logits"]).view(torch.bfloat16).float().numpy()
    got = to_f32(out[ir["graph_outputs"][0]["name"]])
    assert np.abs(got - gold).max() < 0.1 and got[0, -1].argmax() == gold[0, -1].argmax()


def test_unfused_generic_path_on_gpu():
    """fuse=False runs every op through the generic kernels (chains, strided copies,
    strided matmul, softmax); it must agree with the fused path and the oracle."""
    from golden.make_golden import tiny_qwen

    cfg, sd, model = tiny_qwen()
    T = 16
    ir = extract_ir(mz.QwenPrefillWrapper(model), mz.qwen2_example_inputs(cfg, 1, T, None, device="cpu"), "p")
    g = torch.Generator().manual_seed(3)
    ins = (torch.randint(0, cfg.vocab_size, (1, T), generator=g), mz.causal_mask(1, T, T, 0), torch.arange(T)[None], torch.arange(T))
    ref = to_f32(list(IRInterpreter(ir, sd).execute(ins).values())[0])
    out, _ = run_backend(ir, mz.state_dict_numpy(sd), np_inputs(ir, ins), {"fuse": False})
    assert np.abs(to_f32(out[ir["graph_outputs"][0]["name"]]) - ref).max() < 0.1


def test_profile_entry_times_one_entry_point_in_a_graph():
    """CUDAExecutor.profile_entry replays the calls of one entry point as a CUDA graph of their own."""
    from golden.make_golden import tiny_qwen

    from cuda_runtime import CUDABuffer

    cfg, sd, model = tiny_qwen()
    T = 16
    ir = extract_ir(mz.QwenPrefillWrapper(model), mz.qwen2_example_inputs(cfg, 1, T, None, device="cpu"), "p")
    g = torch.Generator().manual_seed(3)
    ins = (torch.randint(0, cfg.vocab_size, (1, T), generator=g), mz.causal_mask(1, T, T, 0), torch.arange(T)[None], torch.arange(T))
    _, dag = run_backend(ir, mz.state_dict_numpy(sd), np_inputs(ir, ins))
    pid = next(iter(dag.npu_programs))
    ex, w = dag._npu_executors[pid], dag._npu_weight_cache[pid]
    feed = {s["name"]: CUDABuffer(t.cuda()) for s, t in zip(ir["graph_inputs"], ins)}
    calls, ms = ex.profile_entry(feed, w, "b200_linear", iters=3)
    assert calls > 0 and 0.0 < ms < 5.0
    assert ex.profile_entry(feed, w, "b200_no_such_entry") == (0, 0.0)


# ----------------------------------------------------------------------------------------------
# Parity at the sizes the benchmark times: the full 28-layer network, batch 64, a cache that a
# real prefill produced, ResNet-50 at batch 32.
# ----------------------------------------------------------------------------------------------
def _host_memory_gb() -> float:
    """Host memory this process may still use: free RAM, capped by the container's cgroup limit."""
    import psutil

    avail = psutil.virtual_memory().available
    try:
        limit = Path("/sys/fs/cgroup/memory.max").read_text().strip()
        if limit != "max":
            used = int(Path("/sys/fs/cgroup/memory.current").read_text())
            avail = min(avail, int(limit) - used)
    except (OSError, ValueError):
        pass
    return avail / 2 ** 30


def _decode_pair(L, B, S):
    """(ir, DAGExecutor on the GPU, oracle interpreter, cfg, input names, output names) for a decode graph."""
    from cuda_compiler import compile_subgraph, is_cuda_op_supported
    from cuda_runtime import CUDABackend
    from npu_compiler import partition
    from npu_runtime import DAGExecutor

    cfg, sd, model = _qwen(L)
    ir = extract_ir(mz.QwenDecodeWrapper(model, L), mz.qwen2_example_inputs(cfg, B, 1, S), "qd")
    dag = DAGExecutor(partition(ir, is_cuda_op_supported), CUDABackend(), compile_subgraph)
    dag.load_weights(mz.state_dict_numpy(sd))
    return ir, dag, IRInterpreter(ir, sd), cfg, [s["name"] for s in ir["graph_inputs"]], [o["name"] for o in ir["graph_outputs"]]


# Logits tolerance of the full-depth network.  bf16 carries 8 significant bits; the GPU kernels
# accumulate in fp32 in another order than ATen's CPU kernels and round at the same points, so
# each layer adds a rounding-level difference to the residual stream.  Two layers measure
# <= 0.1 on logits of magnitude ~4 (bound 0.15 above); 28 layers are bounded by 0.3 absolute
# and 7.5 % of the largest logit, both asserted (measured: 0.20 for one step, 0.24 after eight
# free-running steps whose cache rows carry the earlier steps' differences).
TOL_28_ABS, TOL_28_REL = 0.3, 0.075


def _check_top5(got, want, err):
    """The reference asks for >= 3 common members between the two top-5 sets
    (tests/test_e2e_qwen.py:126-137), on a trained checkpoint whose logits are peaked.  The seeded
    random weights used here give nearly flat logits (the oracle's 1st and 6th largest are ~0.15
    apart, about the bf16 error of a 28-layer network), so the check is made error-aware: every
    member of the GPU's top-5 must lie within 2 x the measured logits error of the oracle's 5th
    largest logit, and fewer than 3 common members are accepted only when the oracle's own 3rd and
    6th largest are that close, i.e. when the set has fewer than 3 stable members.  Returns the
    smallest overlap seen."""
    worst = 5
    for b in range(got.shape[0]):
        order = np.argsort(-want[b])
        g5 = np.argsort(-got[b])[:5]
        fifth = want[b][order[4]]
        assert all(want[b][j] >= fifth - 2 * err for j in g5), (b, [float(want[b][j]) for j in g5], float(fifth), err)
        ov = len(set(g5.tolist()) & set(order[:5].tolist()))
        if ov < 3:
            assert want[b][order[2]] - want[b][order[5]] < 2 * err, (b, ov, want[b][order[:6]], err)
        worst = min(worst, ov)
    return worst


def _check_tokens(got, want, err):
    """Arg-max tokens must agree; a disagreement is a tie only if the oracle's own top-2 gap is
    below twice the measured logits error.  Returns the number of ties."""
    ties = 0
    for b in range(got.shape[0]):
        if got[b].argmax() != want[b].argmax():
            top2 = np.sort(want[b])[-2:]
            assert top2[1] - top2[0] < 2 * err, (b, got[b].argmax(), want[b].argmax(), top2, err)
            ties += 1
    return ties


def test_qwen_28_layers_free_running_greedy_decode_matches_oracle():
    """The whole 28-layer network, B=8, eight greedy steps in which the GPU feeds its own arg-max
    token back (free running).  The oracle follows the same token sequence with its own caches, so
    every step compares logits, tokens and the cache row written."""
    from cuda_runtime import CUDABuffer

    L, B, S, P, steps = 28, 8, 4352, 4096, 8
    ir, dag, interp, cfg, names_in, names_out = _decode_pair(L, B, S)
    g = torch.Generator().manual_seed(5)
    kv = [(torch.randn(B, 2, S, 128, generator=g) * 0.5).bfloat16() for _ in range(2 * L)]
    ids = torch.randint(0, cfg.vocab_size, (B, 1), generator=g)
    dev_kv = [CUDABuffer.from_numpy(torch_to_numpy(t)) for t in kv]
    ref_kv = list(kv)
    ties, worst, min_overlap = 0, 0.0, 5
    for step in range(steps):
        pos = P + step
        fixed = (mz.causal_mask(B, 1, S, pos), torch.full((B, 1), pos), torch.tensor([pos]))
        out = dag.execute(dict(zip(names_in, [ids.numpy()] + [torch_to_numpy(t) for t in fixed] + dev_kv)))
        ref = interp.execute((ids, *fixed, *ref_kv))
        got, want = to_f32(out[names_out[0]])[:, 0], to_f32(ref[names_out[0]])[:, 0]
        err = float(np.abs(got - want).max())
        worst = max(worst, err)
        assert err < TOL_28_ABS and err < TOL_28_REL * float(np.abs(want).max()), (step, err, float(np.abs(want).max()))
        min_overlap = min(min_overlap, _check_top5(got, want, err))
        ties += _check_tokens(got, want, err)
        # last layer's key cache: the row written in this step is close, every untouched row bit-identical
        k_last, k_ref = out[names_out[-2]].to_numpy(), torch_to_numpy(ref[names_out[-2]])
        untouched = np.ones(S, bool)
        untouched[P:pos + 1] = False
        np.testing.assert_array_equal(k_last.view(np.uint16)[:, :, untouched], k_ref.view(np.uint16)[:, :, untouched])
        # (key rows of the LAST layer carry the accumulated rounding differences of 27 layers: values ~2, bound 0.2)
        assert np.abs(to_f32(k_last[:, :, P:pos + 1]) - to_f32(k_ref[:, :, P:pos + 1])).max() < 0.2
        ids = torch.from_numpy(got.argmax(-1))[:, None]        # the GPU's own token goes back in
        dev_kv = [out[n] for n in names_out[1:]]
        ref_kv = [ref[n] for n in names_out[1:]]
    print(f"28 layers, B={B}, {steps} free-running steps: worst logits error {worst:.4f} (max |logit| {float(np.abs(want).max()):.2f}), "
          f"{ties} tie(s) of {B * steps} tokens, smallest top-5 overlap {min_overlap}")


def test_qwen_28_layers_batch_64_step_matches_oracle():
    """One step of exactly the graph the benchmark times: 28 layers, 64 sequences, cache 4352 / 4096."""
    from cuda_runtime import CUDABuffer

    L, B, S, P = 28, 64, 4352, 4096
    if _host_memory_gb() < 40:   # the oracle holds the 8 GB cache twice (out-of-place index_copy) plus weights
        pytest.skip(f"the CPU oracle needs ~30 GB of host memory for this case, {_host_memory_gb():.0f} GB available")
    ir, dag, interp, cfg, names_in, names_out = _decode_pair(L, B, S)
    g = torch.Generator().manual_seed(6)
    kv = [(torch.randn(B, 2, S, 128, generator=g) * 0.5).bfloat16() for _ in range(2 * L)]
    ids = torch.randint(0, cfg.vocab_size, (B, 1), generator=g)
    fixed = (mz.causal_mask(B, 1, S, P), torch.full((B, 1), P), torch.tensor([P]))
    out = dag.execute(dict(zip(names_in, [ids.numpy()] + [torch_to_numpy(t) for t in fixed] + [CUDABuffer.from_numpy(torch_to_numpy(t)) for t in kv])))
    ref = interp.execute((ids, *fixed, *kv))
    got, want = to_f32(out[names_out[0]])[:, 0], to_f32(ref[names_out[0]])[:, 0]
    err = float(np.abs(got - want).max())
    assert err < TOL_28_ABS and err < TOL_28_REL * float(np.abs(want).max()), (err, float(np.abs(want).max()))
    overlap = [_check_top5(got, want, err)]
    ties = _check_tokens(got, want, err)
    for n in (names_out[1], names_out[-1]):   # first key cache, last value cache: new row close, the rest untouched
        a, b = out[n].to_numpy(), torch_to_numpy(ref[n])
        untouched = np.ones(S, bool)
        untouched[P] = False
        np.testing.assert_array_equal(a.view(np.uint16)[:, :, untouched], b.view(np.uint16)[:, :, untouched])
        assert np.abs(to_f32(a[:, :, P]) - to_f32(b[:, :, P])).max() < 0.2
    print(f"28 layers, B=64 step: logits error {err:.4f} (max |logit| {float(np.abs(want).max()):.2f}), min top-5 overlap {min(overlap)}, {ties} tie(s)")


def test_qwen_prefill_then_decode_on_the_prefilled_cache():
    """Prefill a 512-token prompt on the GPU, hand its K/V to the decode graph's 4352-row caches on
    the device (the reference pads on the host and uploads again, examples/run_qwen.py:132-147),
    then decode greedily; the oracle does the same on the host."""
    from cuda_compiler import compile_subgraph, is_cuda_op_supported
    from cuda_runtime import CUDABackend
    from npu_compiler import partition
    from npu_runtime import DAGExecutor
    from qwen_session import hand_off_kv, kv_mapping

    L, T, S, steps = 4, 512, 4352, 4
    cfg, sd, model = _qwen(L)
    irp = extract_ir(mz.QwenPrefillWrapper(model), mz.qwen2_example_inputs(cfg, 1, T, None), "qp")
    ird = extract_ir(mz.QwenDecodeWrapper(model, L), mz.qwen2_example_inputs(cfg, 1, 1, S), "qd")
    mapping = kv_mapping(irp, ird, L, T, S)
    backend = CUDABackend()
    w = mz.state_dict_numpy(sd)
    dp, dd = (DAGExecutor(partition(ir, is_cuda_op_supported), backend, compile_subgraph) for ir in (irp, ird))
    dp.load_weights(w)
    dd.load_weights(w)
    g = torch.Generator().manual_seed(9)
    pins = (torch.randint(0, cfg.vocab_size, (1, T), generator=g), mz.causal_mask(1, T, T, 0), torch.arange(T)[None], torch.arange(T))
    pre = dp.execute(np_inputs(irp, pins))
    pre_ref = IRInterpreter(irp, sd).execute(pins)
    pn = [o["name"] for o in irp["graph_outputs"]]
    lg, lw = to_f32(pre[pn[0]])[0, -1], to_f32(pre_ref[pn[0]])[0, -1]
    err = float(np.abs(to_f32(pre[pn[0]]) - to_f32(pre_ref[pn[0]])).max())
    assert err < 0.15
    _check_tokens(lg[None], lw[None], err)
    ids = torch.tensor([[int(lg.argmax())]])
    # device-side hand-off against the host statement of it
    dev_kv = hand_off_kv(pre, mapping, ird, backend)
    ref_kv = {}
    for layer in mapping["layers"]:
        for pk, dk in ((layer["prefill_key_output"], layer["decode_key_input"]), (layer["prefill_value_output"], layer["decode_value_input"])):
            buf = torch.zeros(1, 2, S, 128, dtype=torch.bfloat16)
            buf[:, :, :T] = pre_ref[pk]
            ref_kv[dk] = buf
            got = dev_kv[dk].to_numpy()
            assert (got.view(np.uint16)[:, :, T:] == 0).all()
            np.testing.assert_array_equal(got.view(np.uint16)[:, :, :T], pre[pk].to_numpy().view(np.uint16))
    interp = IRInterpreter(ird, sd)
    dn_in, dn_out = [s["name"] for s in ird["graph_inputs"]], [o["name"] for o in ird["graph_outputs"]]
    kv_in_names = dn_in[4:]
    ties = 0
    for step in range(steps):
        pos = T + step
        fixed = (mz.causal_mask(1, 1, S, pos), torch.full((1, 1), pos), torch.tensor([pos]))
        feed = dict(zip(dn_in[:4], [ids.numpy()] + [torch_to_numpy(t) for t in fixed]))
        feed.update(dev_kv)
        out = dd.execute(feed)
        ref = interp.execute((ids, *fixed, *[ref_kv[n] for n in kv_in_names]))
        got, want = to_f32(out[dn_out[0]])[:, 0], to_f32(ref[dn_out[0]])[:, 0]
        err = float(np.abs(got - want).max())
        assert err < 0.15, (step, err)
        ties += _check_tokens(got, want, err)
        ids = torch.from_numpy(got.argmax(-1))[:, None]
        dev_kv = dict(zip(kv_in_names, [out[n] for n in dn_out[1:]]))
        ref_kv = dict(zip(kv_in_names, [ref[n] for n in dn_out[1:]]))
    print(f"prefill {T} -> decode {steps} steps: {ties} tie(s)")


def test_resnet50_batch_32_vs_fp32_oracle():
    """ResNet-50 at the batch size where the persistent convolution kernel, resident weights and wide
    tiles are chosen.  The reference's bound for this network is 2e-1 absolute on logits of magnitude
    ~10 (tests/test_e2e_resnet.py:267-271), i.e. 2 % of the largest logit; the seeded initialisation
    here gives logits in the hundreds, so the bound is asserted in that relative form, explicitly."""
    m = mz.resnet(50, seed=0)
    x = torch.randn(32, 3, 224, 224, generator=torch.Generator().manual_seed(2))
    ir = extract_ir(m, (x,), "resnet50")
    ref = to_f32(list(IRInterpreter(ir, m.state_dict()).execute({"x": x}).values())[0])
    out, _ = run_backend(ir, mz.state_dict_numpy(m.state_dict()), {"x": x.numpy()})
    got = to_f32(out[ir["graph_outputs"][0]["name"]])
    assert np.isfinite(got).all()
    rel = float(np.abs(got - ref).max() / np.abs(ref).max())
    assert rel <= 2e-2, rel
    assert (got.argmax(-1) == ref.argmax(-1)).all()
    overlap = [len(set(np.argsort(-got[b])[:5]) & set(np.argsort(-ref[b])[:5])) for b in range(32)]
    assert min(overlap) >= 4, overlap
    print(f"ResNet-50 b32: max|d|/max|ref| = {rel:.5f} (max|ref| {np.abs(ref).max():.1f}), min top-5 overlap {min(overlap)}")


def test_mixed_device_and_host_partitions_with_pinned_transfers():
    """An op forced to the host (docs/partitioning.md:33-40 of the reference) splits the plan into device -
    host - device partitions; tensors cross the boundaries through page-locked staging buffers.  The mixed
    plan must give what the all-device plan gives."""
    from cuda_compiler import compile_subgraph, is_cuda_op_supported
    from cuda_runtime import CUDABackend
    from cuda_runtime.cuda_backend import staging
    from npu_compiler import partition
    from npu_runtime import DAGExecutor
    from oracle.ir_interpreter import cpu_executor_factory   # stands in for the third-party host interpreter

    m = mz.resnet(18, seed=0)
    x = torch.randn(4, 3, 224, 224, generator=torch.Generator().manual_seed(3))
    ir = extract_ir(m, (x,), "resnet18")
    w = mz.state_dict_numpy(m.state_dict())
    name = ir["graph_outputs"][0]["name"]
    all_dev, _ = run_backend(ir, w, {"x": x.numpy()})
    plan = partition(ir, lambda op, attrs=None: op != "aten.max_pool2d.default" and is_cuda_op_supported(op, attrs))
    kinds = [getattr(s, "target", "transfer") for s in plan.steps]
    assert kinds.count("cpu") == 1 and kinds.count("npu") == 2
    dag = DAGExecutor(plan, CUDABackend(), compile_subgraph, cpu_executor_factory=cpu_executor_factory)
    before = (staging().uploads, staging().downloads)
    out = dag.execute({"x": x.numpy()}, weights=w)
    got = to_f32(out[name])
    assert staging().uploads > before[0] and staging().downloads > before[1]
    ref = to_f32(all_dev[name])
    assert np.abs(got - ref).max() <= 2e-2 * np.abs(ref).max() and (got.argmax(-1) == ref.argmax(-1)).all()
