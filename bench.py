"""Headline benchmark: Qwen2.5-1.5B-architecture greedy decode in bf16 on B200.

One step = one lock-step decode token for B concurrent sequences over a 4352-row KV
cache with 4096 rows already filled (then 4097, ...), through the whole 28-layer graph:
IR -> compile_subgraph -> CUDAExecutor (CUDA graph replay of hand-written kernels) ->
arg-max on the device.  Requests are independent, so with N GPUs every rank serves its
own B sequences with replicated weights and no collective on the data path (weak scaling).

Prints ONE JSON line.  ``--impl reference`` times the reference's CPU path (ATen execution
of the same IR, same batch) on the host cores instead.
"""

from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
for p in (ROOT / "pytorch-apple_b200", ROOT):
    if str(p) not in sys.path:
        sys.path.insert(0, str(p))

import numpy as np  # noqa: E402
import torch  # noqa: E402

import model_zoo as mz  # noqa: E402
from ir_export import extract_ir  # noqa: E402

METRIC = "qwen2.5-1.5b_decode_tokens_per_s"
CACHE_LEN, PREFILLED, LAYERS = 4352, 4096, 28
# dram__bytes_read.sum + dram__bytes_write.sum of one attn_decode_kernel launch at B=64, L=4097, from an
# ncu capture of that launch: 1.02 x the algorithmic bytes, i.e. nothing is read twice.  DRAM counters
# cannot be read without the profiler, so the figure is carried as a constant and only reported for
# the shape it was captured on.
ATTN_DRAM_BYTES_PER_LAUNCH = 274_500_000


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--batch", type=int, default=64, help="sequences per GPU")
    ap.add_argument("--layers", type=int, default=LAYERS)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-extras", action="store_true", help="skip the secondary workloads (prefill, B=1/8 decode, ResNet-50)")
    ap.add_argument("--cpu-sample-batch", type=int, default=8, help="sequences per step of the in-run cpu_baseline sample (b200 arm, N=1)")
    return ap.parse_args()


def measured_peaks():
    f = ROOT / "MEASURED_PEAKS.json"
    if f.exists():
        d = json.loads(f.read_text())
        return d.get("hbm_gbs", 6650.0), d.get("bf16_tflops", 1590.0), "measured"
    return 6650.0, 1590.0, "fallback"


class ClockSampler:
    """nvidia-smi clocks / throttle reasons sampled while the timed region runs."""

    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    PERIOD_MS = int(os.environ.get("B200NN_BENCH_CLOCK_MS", "100"))

    def __init__(self, device_index: int, enabled: bool = True):
        self.idx, self.proc, self.enabled, self.t_mark, self.t_start = device_index, None, enabled, None, None

    def mark(self):
        """The timed region starts now: samples taken earlier are dropped."""
        self.t_mark = time.perf_counter()

    def __enter__(self):
        if not self.enabled:
            return self
        self.t_start = time.perf_counter()
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", str(self.PERIOD_MS),
                                          "-i", str(self.idx)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None
        return self

    def __exit__(self, *exc):
        self.result = {"sm_mhz": None, "sm_max_mhz": None, "reasons": []}
        if self.proc is None:
            return
        time.sleep(0.15)
        self.proc.terminate()
        try:
            text, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            text = ""
        sm, mx, reasons = [], [], set()
        lines = text.splitlines()
        if self.t_mark is not None and self.t_start is not None and lines:
            # samples arrive every 100 ms; keep those of the timed region (the last ones), at least three
            timed = max(3, int((time.perf_counter() - self.t_mark) * 1e3 / self.PERIOD_MS) + 1)
            lines = lines[-timed:]
        for line in lines:
            f = [x.strip() for x in line.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1])); mx.append(float(f[2]))
            except ValueError:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        if sm:
            self.result = {"sm_mhz": float(np.median(sm)), "sm_max_mhz": float(max(mx)), "reasons": sorted(reasons), "samples": len(sm)}


def max_over_ranks(values, world: int, device=None):
    """Slowest rank decides: element-wise MAX of per-rank timings over the process group."""
    if world <= 1:
        return [float(v) for v in values]
    t = torch.tensor(list(values), device=device, dtype=torch.float64)
    torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
    return [float(v) for v in t]


def whole_job_throughput(world: int, units_per_rank_per_step: int, steps: int, ms: float) -> float:
    """Units all ranks processed divided by the (max-over-ranks) time."""
    return world * units_per_rank_per_step * steps / (ms / 1e3)


# ---------------------------------------------------------------------------------------
def decode_bytes_per_step(cfg, B: int, L: int) -> dict:
    """Algorithmic HBM bytes of one decode step: every weight once (tied head counted once,
    embedding gather is B rows), K and V rows 0..L of every layer per sequence, new KV rows."""
    H, I, V = cfg.hidden_size, cfg.intermediate_size, cfg.vocab_size
    kvd = cfg.num_key_value_heads * 128
    per_layer = H * H * 2 + 2 * kvd * H + 3 * H * I + H + 2 * kvd + 2 * H
    weights = (cfg.num_hidden_layers * per_layer + V * H + H) * 2
    kv = cfg.num_hidden_layers * 2 * kvd * L * 2 * B
    return {"weights": weights, "kv": kv, "total": weights + kv + cfg.num_hidden_layers * 2 * kvd * 2 * B}


def build_decode(cfg, B: int, device):
    """(ir, dag, argmax executor pieces, weights) for the decode graph on ``device``."""
    from cuda_compiler import compile_subgraph, is_cuda_op_supported
    from cuda_runtime import CUDABackend, CUDABuffer
    from npu_compiler import partition
    from npu_runtime import DAGExecutor

    L = cfg.num_hidden_layers
    ir = extract_ir(mz.QwenDecodeWrapper(mz.qwen2_model(cfg), L), mz.qwen2_example_inputs(cfg, B, 1, CACHE_LEN), "qwen2_decode")
    backend = CUDABackend(device.index)
    dag = DAGExecutor(partition(ir, is_cuda_op_supported), backend, compile_subgraph)
    sd = mz.qwen2_weights(cfg, seed=0, device=str(device))
    dag.load_weights({k: CUDABuffer(v) for k, v in sd.items()})
    V = cfg.vocab_size
    am_ir = {"model_name": "greedy", "graph_inputs": [{"name": "logits", "shape": [B, 1, V], "dtype": "bfloat16"}],
             "graph_outputs": [{"name": "token", "shape": [B, 1], "dtype": "int64"}], "weights": [], "weight_name_mapping": {},
             "nodes": [{"name": "token", "op_type": "aten.argmax.default", "inputs": [{"name": "logits", "shape": [B, 1, V], "dtype": "bfloat16"}],
                        "outputs": [{"name": "token", "shape": [B, 1], "dtype": "int64"}], "attrs": {"dim": -1, "keepdim": False}}]}
    am = DAGExecutor(partition(am_ir, is_cuda_op_supported), backend, compile_subgraph)
    am.load_weights({})
    return ir, dag, am, sd


def run_b200(args, rank: int, world: int, device):
    from cuda_runtime import CUDABuffer
    from cuda_runtime.cuda_backend import torch_to_numpy

    cfg = mz.qwen2_config(num_layers=args.layers)
    B, K, W = args.batch, args.steps, args.warmup
    ir, dag, am, sd = build_decode(cfg, B, device)
    names_in = [s["name"] for s in ir["graph_inputs"]]
    names_out = [o["name"] for o in ir["graph_outputs"]]
    g = torch.Generator(device=device).manual_seed(1234 + rank)
    kv = [CUDABuffer((torch.randn(B, cfg.num_key_value_heads, CACHE_LEN, 128, generator=g, device=device) * 0.5).bfloat16())
          for _ in range(2 * cfg.num_hidden_layers)]
    n_total = K + W
    # host-side step inputs (pinned), as a serving loop would have them
    def host_inputs(i):
        pos = PREFILLED + (i % (CACHE_LEN - PREFILLED))
        return pos, {"attention_mask": torch_to_numpy(mz.causal_mask(B, 1, CACHE_LEN, pos)),
                     "position_ids": np.full((B, 1), pos, np.int64), "cache_position": np.array([pos], np.int64)}

    pid = next(iter(dag.npu_programs))
    executor, weights = dag._npu_executors[pid], dag._npu_weight_cache[pid]
    am_exec = am._npu_executors[next(iter(am.npu_programs))]

    # ---------------- device-resident arm: inputs already in HBM ------------------------
    ids = torch.randint(0, cfg.vocab_size, (B, 1), device=device, generator=g)
    step_in = []
    for i in range(n_total):
        pos, h = host_inputs(i)
        step_in.append({k: torch.from_numpy(v.view(np.uint16) if v.dtype.name == "bfloat16" else v).to(device) for k, v in h.items()})
        step_in[-1]["attention_mask"] = step_in[-1]["attention_mask"].view(torch.bfloat16)
    bufs = {"input_ids": CUDABuffer(ids.clone())}
    for k, t in step_in[0].items():
        bufs[k] = CUDABuffer(t.clone())
    feed = dict(bufs)
    feed.update(dict(zip(names_in[4:], kv)))

    def device_step(i):
        for k, t in step_in[i].items():
            bufs[k].native_handle.copy_(t)
        out = executor.run(feed, weights)
        tok = am_exec.run({"logits": out[names_out[0]]}, {})["token"]
        bufs["input_ids"].native_handle.copy_(tok.native_handle.view(B, 1))
        return out

    # Clocks are sampled by rank 0 only, and the sampler is started before the warm-up: nvidia-smi
    # initialises NVML for every GPU of the box when it starts, which stalls running kernels for a
    # moment (with one sampler per rank inside the timed region, four ranks lost 9 % of a 32-step run).
    with ClockSampler(device.index, enabled=rank == 0) as clocks:
        if rank == 0:
            time.sleep(1.0)   # let nvidia-smi finish starting up
        for i in range(W):
            device_step(i)
        if world > 1:
            torch.distributed.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        clocks.mark()
        e0.record()
        for i in range(W, n_total):
            device_step(i)
        e1.record()
        torch.cuda.synchronize()
    ms = e0.elapsed_time(e1)
    launches_per_step = executor.last_launch_count + am_exec.last_launch_count

    # ---------------- end-to-end arm: host buffers in, token ids out ----------------------
    pinned = []
    for i in range(n_total):
        _, h = host_inputs(i)
        row = {}
        for k, v in h.items():
            t = torch.from_numpy(v.view(np.uint16) if v.dtype.name == "bfloat16" else v).pin_memory()
            row[k] = t.numpy().view(v.dtype) if v.dtype.name == "bfloat16" else t.numpy()
            pinned.append(t)
        step_host = row
        step_in[i] = step_host
    tok_host = torch.randint(0, cfg.vocab_size, (B, 1)).pin_memory()
    kv_feed = dict(zip(names_in[4:], kv))
    h2d = tok_host.numel() * 8 + sum(v.nbytes for v in step_in[0].values())
    d2h = B * 8

    def e2e_step(i, ids_np):
        feed_h = {"input_ids": ids_np, **step_in[i], **kv_feed}
        out = dag.execute(feed_h)
        tok = am.execute({"logits": out[names_out[0]]})["token"].to_numpy()   # device -> host read of the result
        for n, o in zip(names_in[4:], names_out[1:]):
            kv_feed[n] = out[o]
        return tok.reshape(B, 1)

    ids_np = tok_host.numpy()
    for i in range(W):
        ids_np = e2e_step(i, ids_np)
    if world > 1:
        torch.distributed.barrier()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    f0, f1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    f0.record()
    for i in range(W, n_total):
        ids_np = e2e_step(i, ids_np)
    f1.record()
    torch.cuda.synchronize()
    e2e_ms = max(f0.elapsed_time(f1), (time.perf_counter() - t0) * 1e3)

    # ---------------- per-kernel timing of one step (events around every launch) -----------
    prof = executor.profile(feed, weights)
    by_fn: dict[str, list[float]] = {}
    for name, t in prof:
        by_fn.setdefault(name, []).append(t)
    # the dominant kernel again, now as a graph of its own launches only (device time, no host gaps)
    attn_calls, attn_ms = executor.profile_entry(feed, weights, "b200_attn_decode")
    if not attn_calls:
        attn_ms = float(np.mean(by_fn.get("b200_attn_decode", [0.0])))
    L_valid = PREFILLED + 1
    kvd = cfg.num_key_value_heads * 128
    attn_bytes = 2 * kvd * L_valid * 2 * B + 2 * B * cfg.num_attention_heads * 128 * 2 + B * CACHE_LEN * 2
    bts = decode_bytes_per_step(cfg, B, L_valid)
    hbm, _, which = measured_peaks()

    ms, e2e_ms = max_over_ranks([ms, e2e_ms], world, device)
    line = {
        "metric": METRIC, "value": whole_job_throughput(world, B, K, ms), "unit": "tokens/s", "n_gpus": world, "steps": K, "warmup": W,
        "ms_per_step": ms / K, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": workload_config(args.layers, B, world),
        "e2e": {"value": whole_job_throughput(world, B, K, e2e_ms), "unit": "tokens/s", "h2d_bytes_per_step": int(h2d), "d2h_bytes_per_step": int(d2h),
                "ms_per_step": e2e_ms / K, "api": "DAGExecutor.execute(host inputs) -> argmax -> to_numpy()"},
        "gpu_launches": int(launches_per_step * K),
        "clocks": clocks.result,
        "roofline": {"bound": "hbm", "kernel": "attn_decode_kernel", "achieved": attn_bytes / (attn_ms * 1e-3) / 1e9 if attn_ms else None,
                     "peak": hbm, "unit": "GB/s", "frac": (attn_bytes / (attn_ms * 1e-3) / 1e9 / hbm) if attn_ms else None,
                     "peak_source": which, "traffic": ATTN_DRAM_BYTES_PER_LAUNCH if B == 64 else None,
                     "bytes_per_launch": int(attn_bytes), "ms_per_launch": attn_ms,
                     "timing": f"CUDA events around replays of a graph holding the step's {attn_calls} attention launches",
                     "step": {"algorithmic_bytes": int(bts["total"]), "achieved_gbs": bts["total"] / (ms / K * 1e-3) / 1e9,
                              "frac": bts["total"] / (ms / K * 1e-3) / 1e9 / hbm}},
        "kernel_ms_one_step": {k: {"launches": len(v), "total_ms": float(np.sum(v))} for k, v in sorted(by_fn.items())},
    }
    return line, cfg, sd


def cpu_oracle_decode(cfg, sd_cpu, batch: int, steps: int, warmup: int):
    """The reference CPU path on the same IR: ATen on the host cores (oracle port)."""
    from oracle.ir_interpreter import IRInterpreter

    L = cfg.num_hidden_layers
    ir = extract_ir(mz.QwenDecodeWrapper(mz.qwen2_model(cfg), L), mz.qwen2_example_inputs(cfg, batch, 1, CACHE_LEN), "qwen2_decode")
    g = torch.Generator().manual_seed(0)
    kv = [(torch.randn(batch, cfg.num_key_value_heads, CACHE_LEN, 128, generator=g) * 0.5).bfloat16() for _ in range(2 * L)]
    interp = IRInterpreter(ir, sd_cpu)
    ids = torch.randint(0, cfg.vocab_size, (batch, 1), generator=g)
    names_out = [o["name"] for o in ir["graph_outputs"]]
    times = []
    for i in range(warmup + steps):
        pos = PREFILLED + i
        t0 = time.perf_counter()
        out = interp.execute((ids, mz.causal_mask(batch, 1, CACHE_LEN, pos), torch.full((batch, 1), pos), torch.tensor([pos]), *kv))
        ids = out[names_out[0]][:, -1].float().argmax(-1, keepdim=True)
        kv = [out[n] for n in names_out[1:]]
        if i >= warmup:
            times.append(time.perf_counter() - t0)
    return batch * len(times) / sum(times), sum(times)


def workload_config(layers: int, B: int, world: int) -> dict:
    """The ``config`` object of the JSON line; both arms describe the same workload."""
    return {"workload": f"Qwen2.5-1.5B-arch greedy decode, {layers} layers, B={B} sequences per GPU, KV cache {CACHE_LEN} rows "
                        f"with {PREFILLED} filled, lock-step positions from {PREFILLED}", "batch_per_gpu": B,
            "cache_len": CACHE_LEN, "prefilled": PREFILLED, "parallelism": f"replicas x{world}, batch sharded, no collective",
            "l2_policy": "inputs larger than L2: every step streams 3.1 GB of weights and the KV cache"}


def host_threads() -> int:
    """All host cores this process may use (torchrun pins OMP_NUM_THREADS to 1; undo that for the CPU arm)."""
    try:
        return max(1, len(os.sched_getaffinity(0)))
    except AttributeError:
        return max(1, os.cpu_count() or 1)


def run_reference(args):
    """--impl reference: the reference's CPU execution of the same decode graph, with the same
    batch per step and the same warm-up count as the other arm."""
    torch.set_num_threads(host_threads())
    cfg = mz.qwen2_config(num_layers=args.layers)
    sd = mz.qwen2_weights(cfg, seed=0)
    tps, total = cpu_oracle_decode(cfg, sd, args.batch, args.steps, args.warmup)
    threads = torch.get_num_threads()
    sample = (f"{args.steps} whole decode steps of all B={args.batch} sequences after {args.warmup} warm-up steps, {args.layers} layers, "
              f"cache {CACHE_LEN}/{PREFILLED}, {total:.1f} s of CPU time")
    return {
        "impl": "reference", "metric": METRIC, "value": tps, "unit": "tokens/s", "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": total / args.steps * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": workload_config(args.layers, args.batch, max(1, args.gpus)),
        "cpu_baseline": {"value": tps, "unit": "tokens/s", "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": tps, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }


def main():
    args = parse()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        if rank == 0:
            print(json.dumps(run_reference(args)), flush=True)
        return
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the kernel library is the only compute path")
    device = torch.device("cuda", local)
    torch.cuda.set_device(device)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        torch.distributed.init_process_group("nccl", device_id=device)
    line, cfg, sd = run_b200(args, rank, world, device)
    if not args.no_extras:
        import bench_extras

        # ResNet-50 fp16, 256 images per GPU, on every rank: aggregate images/s at this N
        rn = bench_extras.resnet50_replicas(device, 256, world)
        if rank == 0:
            line["also"] = {"resnet50_b256": rn}
            line["also"].update(bench_extras.run(cfg, sd, device))
    if rank == 0:
        if not args.no_cpu_baseline and world == 1:
            # Only at N=1: under torchrun the other ranks would be spinning at the barrier on the same host cores.
            torch.set_num_threads(host_threads())
            sd_cpu = {k: v.cpu() for k, v in sd.items()}
            b = min(args.cpu_sample_batch, args.batch)
            tps, total = cpu_oracle_decode(cfg, sd_cpu, b, 3, 1)
            line["cpu_baseline"] = {"value": tps, "unit": "tokens/s", "cores": torch.get_num_threads(), "kind": "port",
                                    "sample": f"3 decode steps of {b} sequences (of the B={args.batch} workload), {args.layers} layers, "
                                              f"cache {CACHE_LEN}/{PREFILLED}, {total:.1f} s of CPU time"}
        print(json.dumps(line), flush=True)
    if world > 1:
        torch.distributed.barrier()
        torch.distributed.destroy_process_group()


if __name__ == "__main__":
    main()
