"""Pieces of the benchmark harness that can be checked without a GPU."""

import bench_extras


def test_log_scale_positions_match_the_reference_protocol():
    # benchmarks/benchmark_qwen.py:50-58 with max_cache_len 32768 and a 128-token prefill: 1, 2, 4, ..., 16384, 32640
    steps = bench_extras.log_scale_steps(32768 - 128)
    assert steps == [1, 2, 4, 8, 16, 32, 64, 128, 256, 512, 1024, 2048, 4096, 8192, 16384, 32640]
    assert bench_extras.log_scale_steps(1) == [1] and bench_extras.log_scale_steps(5) == [1, 2, 4, 5]
