"""Secondary workloads reported next to the headline decode number (``"also"`` in the
benchmark's JSON line): Qwen2.5-1.5B-architecture decode at B=1 and B=8, prefill of a
512-token prompt, ResNet-50 fp16 inference at batch 1 / 32 / 256, and the bandwidth
kernels (RMSNorm, SiLU*up, masked softmax, RoPE) on their own at 128 / 2048 / 8192 tokens.
All are timed with CUDA events over device-resident inputs, after warm-up, as whole-graph
replays.
"""

from __future__ import annotations

import sys
from pathlib import Path

import numpy as np
import torch

_ROOT = Path(__file__).resolve().parent
for _p in (_ROOT / "pytorch-apple_b200", _ROOT):
    if str(_p) not in sys.path:
        sys.path.insert(0, str(_p))

import model_zoo as mz  # noqa: E402
from ir_export import extract_ir  # noqa: E402

CACHE_LEN, PREFILLED = 4352, 4096


def _time_runs(fn, warmup: int, iters: int) -> float:
    """median milliseconds of ``fn()``"""
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    times = []
    for _ in range(iters):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        torch.cuda.synchronize()
        times.append(a.elapsed_time(b))
    return float(np.median(times))


def _dag(ir, weights, device):
    from cuda_compiler import compile_subgraph, is_cuda_op_supported
    from cuda_runtime import CUDABackend
    from npu_compiler import partition
    from npu_runtime import DAGExecutor

    dag = DAGExecutor(partition(ir, is_cuda_op_supported), CUDABackend(device.index), compile_subgraph)
    dag.load_weights(weights)
    pid = next(iter(dag.npu_programs))
    return dag, dag._npu_executors[pid], dag._npu_weight_cache[pid]


def qwen_decode(cfg, sd, device, B: int, hbm_gbs: float) -> dict:
    from bench import decode_bytes_per_step
    from cuda_runtime import CUDABuffer

    L = cfg.num_hidden_layers
    ir = extract_ir(mz.QwenDecodeWrapper(mz.qwen2_model(cfg), L), mz.qwen2_example_inputs(cfg, B, 1, CACHE_LEN), "qwen2_decode")
    _, ex, w = _dag(ir, {k: CUDABuffer(v) for k, v in sd.items()}, device)
    g = torch.Generator(device=device).manual_seed(7)
    names = [s["name"] for s in ir["graph_inputs"]]
    feed = {"input_ids": CUDABuffer(torch.randint(0, cfg.vocab_size, (B, 1), device=device, generator=g)),
            "attention_mask": CUDABuffer(mz.causal_mask(B, 1, CACHE_LEN, PREFILLED).to(device)),
            "position_ids": CUDABuffer(torch.full((B, 1), PREFILLED, device=device)),
            "cache_position": CUDABuffer(torch.tensor([PREFILLED], device=device))}
    for n in names[4:]:
        feed[n] = CUDABuffer((torch.randn(B, cfg.num_key_value_heads, CACHE_LEN, 128, generator=g, device=device) * 0.5).bfloat16())
    ms = _time_runs(lambda: ex.run(feed, w), 5, 30)
    bts = decode_bytes_per_step(cfg, B, PREFILLED + 1)["total"]
    return {"tokens_per_s": B / (ms / 1e3), "ms_per_step": ms, "algorithmic_bytes": int(bts),
            "hbm_frac": bts / (ms * 1e-3) / 1e9 / hbm_gbs, "launches": ex.last_launch_count}


def qwen_prefill(cfg, sd, device, T: int, tflops_peak: float) -> dict:
    from cuda_runtime import CUDABuffer

    ir = extract_ir(mz.QwenPrefillWrapper(mz.qwen2_model(cfg)), mz.qwen2_example_inputs(cfg, 1, T, None), "qwen2_prefill")
    _, ex, w = _dag(ir, {k: CUDABuffer(v) for k, v in sd.items()}, device)
    g = torch.Generator(device=device).manual_seed(7)
    feed = {"input_ids": CUDABuffer(torch.randint(0, cfg.vocab_size, (1, T), device=device, generator=g)),
            "attention_mask": CUDABuffer(mz.causal_mask(1, T, T, 0).to(device)),
            "position_ids": CUDABuffer(torch.arange(T, device=device)[None]),
            "cache_position": CUDABuffer(torch.arange(T, device=device))}
    ms = _time_runs(lambda: ex.run(feed, w), 3, 10)
    H, I, V, L = cfg.hidden_size, cfg.intermediate_size, cfg.vocab_size, cfg.num_hidden_layers
    kvd = cfg.num_key_value_heads * 128
    flops = 2 * T * (L * (H * H * 2 + 2 * kvd * H + 3 * H * I) + V * H) + L * cfg.num_attention_heads * 4 * T * T * 128
    return {"ms": ms, "tflops": flops / (ms * 1e-3) / 1e12, "tensor_frac": flops / (ms * 1e-3) / 1e12 / tflops_peak,
            "algorithmic_flops": int(flops), "launches": ex.last_launch_count, "tokens": T,
            "launches_are": "library calls (a down projection split over CTA pairs is two kernels inside one call)"}


def resnet50(device, batch: int, tflops_peak: float) -> dict:
    from cuda_runtime import CUDABuffer

    m = mz.resnet(50, seed=0)
    ir = extract_ir(mz.resnet(50, device="meta"), (torch.zeros(batch, 3, 224, 224, device="meta"),), "resnet50")
    _, ex, w = _dag(ir, mz.state_dict_numpy(m.state_dict()), device)
    x = torch.randn(batch, 3, 224, 224, device=device, generator=torch.Generator(device=device).manual_seed(0)).half()
    feed = {ir["graph_inputs"][0]["name"]: CUDABuffer(x)}
    ms = _time_runs(lambda: ex.run(feed, w), 5, 20)
    flops = 8.178e9 * batch
    return {"images_per_s": batch / (ms / 1e3), "ms": ms, "tflops": flops / (ms * 1e-3) / 1e12,
            "tensor_frac": flops / (ms * 1e-3) / 1e12 / tflops_peak, "launches": ex.last_launch_count}


def resnet50_replicas(device, batch: int, world: int) -> dict:
    """ResNet-50 on every rank at once (replicated weights, ``batch`` images per GPU, no collective on
    the data path): whole-job images/s = world * batch / the slowest rank's time."""
    from bench import max_over_ranks, measured_peaks

    _, tf, _ = measured_peaks()
    if world > 1:
        torch.distributed.barrier()
    res = resnet50(device, batch, tf)
    ms = max_over_ranks([res["ms"]], world, device)[0]
    flops = 8.178e9 * batch
    return {"images_per_s": world * batch / (ms / 1e3), "ms": ms, "n_gpus": world, "batch_per_gpu": batch,
            "tflops_per_gpu": flops / (ms * 1e-3) / 1e12, "tensor_frac": flops / (ms * 1e-3) / 1e12 / tf,
            "launches": res["launches"], "timing": "median of 20 graph replays per rank, max over ranks"}


# (in channels, input size, out channels, kernel, stride, padding, residual, how many) - the
# distinct convolutions of ResNet-50 at 224 x 224 (the stem with its input padded to 8 channels)
RESNET50_CONVS = [
    (8, 224, 64, 7, 2, 3, 0, 1),
    (64, 56, 64, 1, 1, 0, 0, 1), (64, 56, 64, 3, 1, 1, 0, 3), (64, 56, 256, 1, 1, 0, 1, 3), (64, 56, 256, 1, 1, 0, 0, 1),
    (256, 56, 64, 1, 1, 0, 0, 2), (256, 56, 128, 1, 1, 0, 0, 1), (128, 56, 128, 3, 2, 1, 0, 1), (128, 28, 512, 1, 1, 0, 1, 4),
    (256, 56, 512, 1, 2, 0, 0, 1), (512, 28, 128, 1, 1, 0, 0, 3), (128, 28, 128, 3, 1, 1, 0, 3), (512, 28, 256, 1, 1, 0, 0, 1),
    (256, 28, 256, 3, 2, 1, 0, 1), (256, 14, 1024, 1, 1, 0, 1, 6), (512, 28, 1024, 1, 2, 0, 0, 1), (1024, 14, 256, 1, 1, 0, 0, 5),
    (256, 14, 256, 3, 1, 1, 0, 5), (1024, 14, 512, 1, 1, 0, 0, 1), (512, 14, 512, 3, 2, 1, 0, 1), (512, 7, 2048, 1, 1, 0, 1, 3),
    (1024, 14, 2048, 1, 2, 0, 0, 1), (2048, 7, 512, 1, 1, 0, 0, 2), (512, 7, 512, 3, 1, 1, 0, 2)]


def resnet50_layers(device, batch: int, hbm_gbs: float, tflops_peak: float) -> list:
    """Every distinct convolution of ResNet-50 on its own through ``b200_conv2d_nhwc`` (fp16,
    NHWC, bias + ReLU, residual where the network has one): microseconds per call (five calls
    back to back, CUDA events) next to its roofline time = max(flops / tensor peak, bytes / HBM peak)."""
    from cuda_runtime import native

    lib = native.load()
    st = torch.cuda.current_stream().cuda_stream
    rows = []
    for cin, h, o, k, s, p, res, count in RESNET50_CONVS:
        ho = (h + 2 * p - k) // s + 1
        x = torch.randn(batch, h, h, cin, device=device).half()
        w = (torch.randn(o, k * k * cin, device=device) * 0.05).half()
        bias = torch.zeros(o, device=device)
        r = torch.randn(batch, ho, ho, o, device=device).half()
        y = torch.empty(batch, ho, ho, o, device=device, dtype=torch.half)

        def call():
            native.check(lib.b200_conv2d_nhwc(x.data_ptr(), w.data_ptr(), bias.data_ptr(), r.data_ptr() if res else None, y.data_ptr(),
                                              batch, h, h, cin, cin, o, k, k, s, s, p, p, ho, ho, 1, 1, st))

        def five():
            for _ in range(5):
                call()

        us = _time_runs(five, 2, 5) / 5 * 1e3
        flops = 2 * batch * ho * ho * o * k * k * cin
        nbytes = 2 * (batch * h * h * cin + batch * ho * ho * o * (2 if res else 1) + o * k * k * cin)
        t_tensor, t_hbm = flops / (tflops_peak * 1e12) * 1e6, nbytes / (hbm_gbs * 1e9) * 1e6
        rows.append({"conv": f"{cin}->{o} {k}x{k}/{s} @{h}" + (" +res" if res else ""), "count": count, "us": round(us, 1),
                     "roofline_us": round(max(t_tensor, t_hbm), 1), "bound": "tensor" if t_tensor > t_hbm else "hbm",
                     "frac": round(max(t_tensor, t_hbm) / us, 2)})
    return rows


def ops(device, hbm_gbs: float, tokens=(128, 2048, 8192)) -> dict:
    """The bandwidth kernels on their own, at Qwen2.5-1.5B widths and ``T`` tokens, bf16:
    RMSNorm [T,1536]; SiLU(gate)*up [T,8960]; masked softmax over [1,12,T,T] scores with a
    [1,1,T,T] additive mask; rotary embedding of q [1,12,T,128].  Each call is captured
    into a CUDA graph that walks enough separate buffer sets to exceed the L2 (so every
    call reads cold data), and the graph is timed with CUDA events.  ``gbs`` is the
    algorithmic bytes of one call (inputs read once, outputs written once) over its share
    of the graph's time."""
    from cuda_compiler.cuda_codegen import EW_OPCODES
    from cuda_runtime import native

    lib = native.load()
    BF = native.DTYPE_CODES["bfloat16"]
    H, I, NH, D = 1536, 8960, 12, 128
    gen = torch.Generator(device=device).manual_seed(3)

    def rnd(*shape):
        return torch.randn(*shape, device=device, generator=gen).bfloat16()

    def timed(bytes_per_call, make_set, call):
        n_sets = int(max(2, min(64, -(-400_000_000 // bytes_per_call))))
        sets = [make_set() for _ in range(n_sets)]
        side = torch.cuda.Stream(device)
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for s in sets:
                call(s, side.cuda_stream)
        side.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=side):
            for s in sets:
                call(s, side.cuda_stream)
        ms = _time_runs(graph.replay, 3, 15) / n_sets
        return {"us": ms * 1e3, "gbs": bytes_per_call / (ms * 1e-3) / 1e9, "hbm_frac": bytes_per_call / (ms * 1e-3) / 1e9 / hbm_gbs,
                "algorithmic_bytes": int(bytes_per_call), "buffer_sets": n_sets}

    out = {}
    for T in tokens:
        res = {}
        w = rnd(H)
        res["rmsnorm"] = timed(2 * T * H * 2 + H * 2, lambda: (rnd(T, H), torch.empty(T, H, device=device, dtype=torch.bfloat16)),
                               lambda s, st: native.check(lib.b200_rmsnorm(s[0].data_ptr(), w.data_ptr(), s[1].data_ptr(), T, H, H, H, 1e-6, BF, 1, st)))
        chain = (native.EwOp * 2)(native.EwOp(EW_OPCODES["SILU"], 0, -1, BF, 0.0), native.EwOp(EW_OPCODES["MUL"], 4, 1, BF, 0.0))

        def silu_mul(s, st):
            ins = (native.Tensor * 2)(*[native.make_tensor(t.data_ptr(), "bfloat16", (T, I), (I, 1)) for t in s[:2]])
            o = native.make_tensor(s[2].data_ptr(), "bfloat16", (T, I), (I, 1))
            native.check(lib.b200_ew_chain(o, ins, 2, chain, 2, st))

        res["silu_mul"] = timed(3 * T * I * 2, lambda: (rnd(T, I), rnd(T, I), torch.empty(T, I, device=device, dtype=torch.bfloat16)), silu_mul)
        mask = torch.full((T, T), float("-inf"), device=device).triu(1).bfloat16()
        res["masked_softmax"] = timed(2 * NH * T * T * 2 + T * T * 2,
                                      lambda: (rnd(NH, T, T), torch.empty(NH, T, T, device=device, dtype=torch.bfloat16)),
                                      lambda s, st: native.check(lib.b200_softmax(s[0].data_ptr(), mask.data_ptr(), s[1].data_ptr(), 1, NH, T, T,
                                                                                   0, 0, T, D ** -0.5, BF, BF, BF, 1, st)))
        cos, sin = rnd(T, D), rnd(T, D)

        def rope(s, st):
            x = native.make_tensor(s[0].data_ptr(), "bfloat16", (1, NH, T, D), (NH * T * D, T * D, D, 1))
            native.check(lib.b200_rope_rotate(x, cos.data_ptr(), sin.data_ptr(), s[1].data_ptr(), None, None, 0, native.DTYPE_CODES["int64"], st))

        res["rope"] = timed(2 * NH * T * D * 2 + 2 * T * D * 2, lambda: (rnd(NH, T, D), torch.empty(NH, T, D, device=device, dtype=torch.bfloat16)), rope)
        out[f"t{T}"] = res
        torch.cuda.empty_cache()
    return out


def log_scale_steps(max_steps: int) -> list[int]:
    """1, 2, 4, ... and max_steps itself: the cache positions the reference's scaling benchmark visits
    (benchmarks/benchmark_qwen.py:50-58)."""
    steps, v = [], 1
    while v < max_steps:
        steps.append(v)
        v *= 2
    return steps + [max_steps]


def decode_sweep(cfg, sd, device, prefill_len: int = 128, max_cache_len: int = 32768, repeats: int = 3) -> dict:
    """The reference's CUDA scaling benchmark (benchmarks/benchmark_qwen.py:650-809) on this backend:
    batch 1, a prefill graph of ``prefill_len`` tokens and a decode graph over a ``max_cache_len``-row
    cache holding random values on the device; for each cache position 1, 2, 4, ... the time of ONE
    decode step through ``DAGExecutor.execute`` with host inputs (ids, mask, positions uploaded every
    call), median of ``repeats``.  One difference, on purpose: the reference reads the clock after the
    call returns without waiting for the GPU (it times the enqueue, :788-793); here the device is
    synchronised before the clock is read, and the device time between two CUDA events is reported too."""
    import time

    from cuda_runtime import CUDABuffer
    from cuda_runtime.cuda_backend import torch_to_numpy

    L = cfg.num_hidden_layers
    weights = {k: CUDABuffer(v) for k, v in sd.items()}
    ir_p = extract_ir(mz.QwenPrefillWrapper(mz.qwen2_model(cfg)), mz.qwen2_example_inputs(cfg, 1, prefill_len, None), "qwen2_prefill")
    ir_d = extract_ir(mz.QwenDecodeWrapper(mz.qwen2_model(cfg), L), mz.qwen2_example_inputs(cfg, 1, 1, max_cache_len), "qwen2_decode")
    dag_p, _, _ = _dag(ir_p, weights, device)
    dag_d, _, _ = _dag(ir_d, weights, device)
    g = torch.Generator().manual_seed(11)
    ids = torch.randint(0, cfg.vocab_size, (1, prefill_len), generator=g)
    pre_in = {"input_ids": ids.numpy(), "attention_mask": torch_to_numpy(mz.causal_mask(1, prefill_len, prefill_len, 0)),
              "position_ids": np.arange(prefill_len, dtype=np.int64)[None], "cache_position": np.arange(prefill_len, dtype=np.int64)}

    def timed(fn, n):
        out = []
        for _ in range(n):
            torch.cuda.synchronize()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            t0 = time.perf_counter()
            a.record()
            fn()
            b.record()
            torch.cuda.synchronize()
            out.append(((time.perf_counter() - t0) * 1e3, a.elapsed_time(b)))
        wall, dev = zip(*out)
        return float(np.median(wall)), float(np.median(dev)), float(np.std(wall))

    for _ in range(3):
        dag_p.execute(pre_in)
    ttft_ms, ttft_dev, _ = timed(lambda: dag_p.execute(pre_in), max(repeats, 7))
    gd = torch.Generator(device=device).manual_seed(12)
    names = [s_["name"] for s_ in ir_d["graph_inputs"]]
    kv = {n: CUDABuffer(torch.randn(1, cfg.num_key_value_heads, max_cache_len, 128, generator=gd, device=device).bfloat16()) for n in names[4:]}

    def step_inputs(cur_pos):
        d = {"input_ids": np.array([[1]], np.int64), "attention_mask": torch_to_numpy(mz.causal_mask(1, 1, max_cache_len, cur_pos)),
             "position_ids": np.array([[cur_pos]], np.int64), "cache_position": np.array([cur_pos], np.int64)}
        d.update(kv)
        return d

    warm = step_inputs(prefill_len)
    for _ in range(3):
        dag_d.execute(warm)
    rows = []
    for pos in log_scale_steps(max_cache_len - prefill_len):
        feed = step_inputs(prefill_len + pos - 1)
        wall, dev, std = timed(lambda: dag_d.execute(feed), repeats)
        rows.append({"position": pos, "step_ms": round(wall, 4), "step_ms_std": round(std, 4), "device_ms": round(dev, 4), "tps": round(1e3 / wall, 1)})
    return {"protocol": f"batch 1, prefill graph {prefill_len} tokens, decode graph over a {max_cache_len}-row cache (random values), "
                        f"median of {repeats} single steps per position, host inputs uploaded per call, device synchronised before the clock is read",
            "layers": L, "ttft_ms": round(ttft_ms, 3), "ttft_device_ms": round(ttft_dev, 3), "points": rows}


def run(cfg, sd, device) -> dict:
    from bench import measured_peaks

    hbm, tf, which = measured_peaks()
    out = {"peaks": {"hbm_gbs": hbm, "bf16_tflops": tf, "source": which}}
    for B in (1, 8):
        out[f"qwen_decode_b{B}"] = qwen_decode(cfg, sd, device, B, hbm)
        torch.cuda.empty_cache()
    out["qwen_prefill_t512"] = qwen_prefill(cfg, sd, device, 512, tf)
    torch.cuda.empty_cache()
    for b in (1, 32):   # batch 256 is measured on every rank by resnet50_replicas
        out[f"resnet50_b{b}"] = resnet50(device, b, tf)
        torch.cuda.empty_cache()
    out["ops"] = ops(device, hbm)
    return out


if __name__ == "__main__":
    # Stand-alone runs of one secondary workload, e.g. for profiling a small case:
    #   python bench_extras.py qwen_prefill --layers 2
    #   python bench_extras.py resnet50 --batch 256
    #   python bench_extras.py qwen_decode --layers 2 --batch 1
    #   python bench_extras.py ops
    #   python bench_extras.py resnet50_layers --batch 256
    #   python bench_extras.py decode_sweep            (the reference's cache-position scaling protocol)
    import argparse
    import json

    from bench import measured_peaks

    ap = argparse.ArgumentParser()
    ap.add_argument("workload", choices=["qwen_prefill", "qwen_decode", "resnet50", "resnet50_layers", "ops", "decode_sweep"])
    ap.add_argument("--layers", type=int, default=28)
    ap.add_argument("--batch", type=int, default=64)
    ap.add_argument("--tokens", type=int, default=512)
    a = ap.parse_args()
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    hbm, tf, _ = measured_peaks()
    if a.workload == "ops":
        print(json.dumps(ops(dev, hbm)))
    elif a.workload == "resnet50_layers":
        rows = resnet50_layers(dev, a.batch, hbm, tf)
        for row in rows:
            print(json.dumps(row))
        print(json.dumps({"sum_us": round(sum(r["us"] * r["count"] for r in rows)),
                          "sum_roofline_us": round(sum(r["roofline_us"] * r["count"] for r in rows))}))
    elif a.workload == "resnet50":
        print(json.dumps(resnet50(dev, a.batch, tf)))
    elif a.workload == "decode_sweep":
        cfg = mz.qwen2_config(num_layers=a.layers)
        sd = mz.qwen2_weights(cfg, seed=0, device=str(dev))
        res = decode_sweep(cfg, sd, dev)
        for row in res["points"]:
            print(json.dumps(row))
        print(json.dumps({k: v for k, v in res.items() if k != "points"}))
    else:
        cfg = mz.qwen2_config(num_layers=a.layers)
        sd = mz.qwen2_weights(cfg, seed=0, device=str(dev))
        res = qwen_prefill(cfg, sd, dev, a.tokens, tf) if a.workload == "qwen_prefill" else qwen_decode(cfg, sd, dev, a.batch, hbm)
        print(json.dumps(res))
