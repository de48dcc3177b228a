"""Parity of every CUDA kernel with a CPU statement of the same op, called through the
C ABI (ctypes on raw device pointers), on seeded inputs.  Integer/byte work must be
bit-exact; floating point uses the op-level tolerance of the reference's CUDA tests
(rtol 5e-2 / atol 1e-2, tests/test_cuda_executor.py:150-319), tightened where bf16 allows."""

import ctypes as C
import math

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

DT = {torch.float32: 0, torch.float16: 1, torch.bfloat16: 2, torch.int32: 3, torch.int64: 4, torch.uint8: 5}


@pytest.fixture(scope="module")
def lib(native_lib):
    assert torch.cuda.is_available()
    torch.cuda.set_device(0)
    return native_lib


def ok(lib, rc):
    assert rc == 0, lib.b200_last_error().decode()
    torch.cuda.synchronize()


def stream():
    return torch.cuda.current_stream().cuda_stream


def gen(shape, dtype=torch.bfloat16, seed=0, scale=1.0):
    return (torch.randn(*shape, generator=torch.Generator().manual_seed(seed)) * scale).to(dtype)


def bt(t):
    from cuda_runtime import native

    return native.make_tensor(t.data_ptr(), str(t.dtype).replace("torch.", ""), tuple(t.shape), tuple(t.stride()))


def close(got, ref, rtol=2e-2, atol=1e-2):
    np.testing.assert_allclose(got.float().cpu().numpy(), ref.float().cpu().numpy(), rtol=rtol, atol=atol)


# ------------------------------------------------------------------ linear
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("M,N,K,bias,res,relu,silu", [
    (1, 1536, 1536, True, False, False, False),
    (1, 1536, 8960, False, True, False, False),
    (8, 8960, 1536, False, False, False, True),
    (64, 256, 1536, True, False, False, False),
    (3, 1000, 512, True, False, True, False),
    (7, 130, 72, True, True, True, False),
    (65, 1536, 1536, True, True, False, False),
    (512, 8960, 1536, False, False, False, True),
    (300, 1000, 2048, True, False, True, False),
    (128, 151936 // 8, 1536, False, False, False, False),
    # 256 x 256 tiles on CTA pairs: row tail (640 = 2 * 256 + 128), column tail, K tail, every epilogue term
    (640, 8200, 1088, True, True, True, False),
    (300, 16384, 1024, True, False, False, False),
    (512, 8960, 1536, True, True, False, True),
    # few 256 x 256 tiles, long reduction: the pairs split K, a second kernel adds the fp32 partial sums
    (1024, 1536, 8960, True, True, False, False),
    (512, 1536, 8960, False, True, False, False),
    (1000, 1200, 4104, False, False, True, False),
])
def test_linear(lib, dtype, M, N, K, bias, res, relu, silu):
    a, w = gen((M, K), dtype), gen((N, K), dtype, 1, 0.05)
    b = gen((N,), dtype, 2) if bias else None
    r = gen((M, N), dtype, 3) if res else None
    u = gen((M, N), dtype, 4) if silu else None
    ref = a.float() @ w.float().t()
    if bias:
        ref = ref + b.float()
    if res:
        ref = ref.to(dtype).float() + r.float()
    if relu:
        ref = torch.relu(ref)
    if silu:
        s = ref.to(dtype).float()
        ref = torch.nn.functional.silu(s).to(dtype).float() * u.float()
    A, W = a.cuda(), w.cuda()
    Bv, Rv, Uv = (t.cuda() if t is not None else None for t in (b, r, u))
    out = torch.full((M, N), float("nan"), dtype=dtype, device="cuda")
    nbytes = lib.b200_linear_workspace_bytes(M, N, K)
    ws = torch.zeros(max(nbytes, 16), dtype=torch.uint8, device="cuda")
    p = lambda t: t.data_ptr() if t is not None else None
    for _ in range(2):  # second call checks that the split-K workspace was left clean
        out.fill_(float("nan"))
        ok(lib, lib.b200_linear(p(A), p(W), p(Bv), p(Rv), p(out), M, N, K, K, K, N, N, DT[dtype], DT[dtype],
                                (1 if relu else 0) | (2 if silu else 0), p(Uv), N, p(ws), ws.numel(), stream()))
        close(out, ref, rtol=2e-2, atol=2e-2 * max(1.0, math.sqrt(K) * 0.05))
    assert not ws.any()
    code = C.c_int(-1)
    ok(lib, lib.b200_debug_device_error(C.byref(code), 1))
    assert code.value == 0, f"a bounded wait in the tcgen05 GEMM gave up (code {code.value})"


@pytest.mark.parametrize("M,N,K", [(128, 128, 64), (129, 200, 72), (1000, 1536, 1536), (512, 151936, 1536)])
def test_linear_tcgen05_shapes(lib, M, N, K):
    """Large-M linears take the tcgen05/TMEM path: tile edges, K tails and a very wide N."""
    dtype = torch.bfloat16
    a, w = gen((M, K), dtype), gen((N, K), dtype, 1, 0.05)
    A, W = a.cuda(), w.cuda()
    out = torch.full((M, N), float("nan"), dtype=dtype, device="cuda")
    ok(lib, lib.b200_linear(A.data_ptr(), W.data_ptr(), None, None, out.data_ptr(), M, N, K, K, K, N, 0, 2, 2, 0, None, 0, None, 0, stream()))
    ref = (A.float() @ W.float().t())           # fp32 GEMM on the device as the large-size reference
    err = (out.float() - ref).abs().max().item()
    assert err <= 2e-2 * max(1.0, math.sqrt(K) * 0.05) + 1e-2 * ref.abs().max().item(), err
    if N <= 2048:
        close(out, a.float() @ w.float().t(), rtol=2e-2, atol=2e-2 * max(1.0, math.sqrt(K) * 0.05))
    code = C.c_int(-1)
    ok(lib, lib.b200_debug_device_error(C.byref(code), 1))
    assert code.value == 0


@pytest.mark.parametrize("M,I,K", [(1, 8960, 1536), (8, 8960, 1536), (64, 8960, 1536), (512, 8960, 1536), (40, 256, 72)])
def test_linear_gated_mlp_epilogue(lib, M, I, K):
    """silu(x Wg^T) * (x Wu^T) from one GEMM over gate/up rows interleaved in blocks of 64."""
    dtype = torch.bfloat16
    x, wg, wu = gen((M, K), dtype), gen((I, K), dtype, 1, 0.05), gen((I, K), dtype, 2, 0.05)
    g = (x.float() @ wg.float().t()).to(dtype).float()
    u = (x.float() @ wu.float().t()).to(dtype).float()
    ref = torch.nn.functional.silu(g).to(dtype).float() * u
    merged = torch.stack([wg.view(I // 64, 64, K), wu.view(I // 64, 64, K)], 1).reshape(2 * I, K).contiguous()
    X, W = x.cuda(), merged.cuda()
    out = torch.full((M, I), float("nan"), dtype=dtype, device="cuda")
    ws = torch.zeros(max(lib.b200_linear_workspace_bytes(M, 2 * I, K), 16), dtype=torch.uint8, device="cuda")
    for _ in range(2):
        ok(lib, lib.b200_linear(X.data_ptr(), W.data_ptr(), None, None, out.data_ptr(), M, 2 * I, K, K, K, I, 0, 2, 2, 4, None, 0,
                                ws.data_ptr(), ws.numel(), stream()))
        close(out, ref, rtol=3e-2, atol=3e-2 * max(1.0, math.sqrt(K) * 0.05))
    assert not ws.any()


@pytest.mark.parametrize("M,N,K,mode", [(1, 2048, 1536, "bias"), (8, 2048, 1536, "bias"), (64, 2048, 1536, "bias"), (64, 17920, 1536, "glu"),
                                        (5, 17920, 1536, "glu"), (64, 151936, 1536, "plain"), (33, 1536, 1536, "chain"), (64, 1536, 8960, "chain")])
def test_linear_norm_fused_rmsnorm(lib, M, N, K, mode):
    """RMSNorm folded into decode GEMMs.  "chain": a residual GEMM that also writes the sum-of-squares
    partials of its output rows, followed by a GEMM over gain-folded weights that scales its output
    rows by 1/rms from those partials - against the fp32 statement of rmsnorm + matmul with the
    roundings of the unfused kernels, and against the unfused kernels themselves."""
    dtype = torch.bfloat16
    BF = 2
    if mode == "chain":
        a, w, res = gen((M, K), dtype, 0, 0.5), gen((N, K), dtype, 1, 0.05), gen((M, N), dtype, 2)
        y = torch.empty(M, N, dtype=dtype, device="cuda")
        sq = torch.full((M, N // 64), float("nan"), device="cuda")
        A, W, R = a.cuda(), w.cuda(), res.cuda()
        ok(lib, lib.b200_linear_norm(A.data_ptr(), W.data_ptr(), None, R.data_ptr(), y.data_ptr(), M, N, K, K, K, N, N, BF, BF, 8,
                                     0.0, None, 0, sq.data_ptr(), stream()))
        ref = ((a.float() @ w.float().T).to(dtype).float() + res.float()).to(dtype)
        close(y, ref, rtol=2e-2, atol=2e-2)
        # the partials describe the rows that were actually written
        want_sq = y.float().pow(2).reshape(M, N // 64, 64).sum(-1)
        torch.testing.assert_close(sq, want_sq, rtol=1e-4, atol=1e-4)
        x, n_part, sumsq = y, N // 64, sq       # feed the next layer from them
        K2, N2 = N, 2048
    else:
        x = gen((M, K), dtype, 0, 3.0).cuda()
        n_part = 3
        sumsq = x.float().pow(2).reshape(M, n_part, K // n_part).sum(-1).contiguous()
        K2, N2 = K, N
    gain = (1 + 0.1 * gen((K2,), torch.float32, 5)).to(dtype).cuda()
    w2 = gen((N2, K2), dtype, 6, 0.03).cuda()
    w2_folded = (w2.float() * gain.float()[None, :]).to(dtype)          # what the weight preparation produces
    bias = gen((N2,), dtype, 7).cuda() if mode in ("bias", "chain") else None
    epi = 8 | (4 if mode == "glu" else 0)
    n_out = N2 // 2 if mode == "glu" else N2
    out = torch.full((M, n_out), float("nan"), dtype=dtype, device="cuda")
    ok(lib, lib.b200_linear_norm(x.data_ptr(), w2_folded.data_ptr(), bias.data_ptr() if bias is not None else None, None, out.data_ptr(), M, N2, K2,
                                 K2, K2, n_out, 0, BF, BF, epi, 1e-6, sumsq.data_ptr(), n_part, None, stream()))

    def finish(r):
        if bias is not None:
            r = r + bias.float().cpu()
        if mode == "glu":
            r = r.reshape(M, N2 // 128, 2, 64)
            g_, u_ = r[:, :, 0].to(dtype).float(), r[:, :, 1].to(dtype).float()
            r = (torch.nn.functional.silu(g_).to(dtype).float() * u_).reshape(M, n_out)
        return r

    xf = x.float().cpu()
    rr = torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + 1e-6)
    # the reference's rounding points: round(x r), round(. * gain), then the GEMM
    a2 = ((xf * rr).to(dtype).float() * gain.float().cpu()).to(dtype).float()
    # (the gated form multiplies two rounded factors: a one-ulp difference in the gate is scaled by |up| <= ~5)
    tol = 6e-2 if mode == "glu" else 3e-2
    close(out, finish(a2 @ w2.float().cpu().T), rtol=3e-2, atol=tol)
    # the exact statement of what the kernel computes: r * (x W'^T)
    close(out, finish(rr * (xf @ w2_folded.float().cpu().T)), rtol=2e-2, atol=tol / 2)
    # and the unfused pair of kernels
    y_n = torch.empty_like(x)
    ok(lib, lib.b200_rmsnorm(x.data_ptr(), gain.data_ptr(), y_n.data_ptr(), M, K2, K2, K2, 1e-6, BF, 1, stream()))
    out2 = torch.empty_like(out)
    ok(lib, lib.b200_linear(y_n.data_ptr(), w2.data_ptr(), bias.data_ptr() if bias is not None else None, None, out2.data_ptr(), M, N2, K2,
                            K2, K2, n_out, 0, BF, BF, epi, None, 0, None, 0, stream()))
    close(out, out2, rtol=3e-2, atol=tol)
    code = C.c_int(0)
    ok(lib, lib.b200_debug_device_error(C.byref(code), 1))
    assert code.value == 0


def test_linear_norm_rejects_shapes_outside_the_fused_kernel(lib):
    t = torch.zeros(128 * 1536, dtype=torch.bfloat16, device="cuda")
    f = torch.zeros(4096, device="cuda")
    args = lambda M, N, K, cols, sq_out: (t.data_ptr(), t.data_ptr(), None, None, t.data_ptr(), M, N, K, K, K, N, 0, 2, 2, 0, 1e-6,
                                          f.data_ptr(), cols, f.data_ptr() if sq_out else None, stream())
    assert lib.b200_linear_norm(*args(100, 64, 128, 1, False)) == -4 and b"M <= 64" in lib.b200_last_error()   # prefill-sized M
    assert lib.b200_linear_norm(*args(8, 64, 128, 40, False)) == -4                                              # too many partials
    assert lib.b200_linear_norm(*args(8, 72, 128, 1, True)) == -4                                                # N not a multiple of 64


def test_bounded_wait_runs_out_and_the_context_survives(lib):
    """A barrier wait that can never be satisfied: the kernel's bounded wait gives up after the probe limit,
    leaves code 99 in the device error word and returns; the next kernels run normally."""
    code = C.c_int(-1)
    ok(lib, lib.b200_debug_device_error(C.byref(code), 1))
    assert code.value == 0
    ok(lib, lib.b200_debug_wait_timeout(2000, stream()))
    ok(lib, lib.b200_debug_device_error(C.byref(code), 0))
    assert code.value == 99
    ok(lib, lib.b200_debug_device_error(C.byref(code), 1))     # reads 99 again and clears
    ok(lib, lib.b200_debug_device_error(C.byref(code), 0))
    assert code.value == 0
    a, w = gen((4, 256)), gen((128, 256), seed=1)
    out = torch.empty(4, 128, dtype=torch.bfloat16, device="cuda")
    A, W = a.cuda(), w.cuda()
    ok(lib, lib.b200_linear(A.data_ptr(), W.data_ptr(), None, None, out.data_ptr(), 4, 128, 256, 256, 256, 128, 0, 2, 2, 0, None, 0, None, 0, stream()))
    close(out, a.float() @ w.float().T, rtol=2e-2, atol=2e-2)
    assert lib.b200_debug_wait_timeout(0, stream()) == -1


def test_linear_rejects_unaligned(lib):
    a = torch.zeros(4, 12, dtype=torch.bfloat16, device="cuda")
    rc = lib.b200_linear(a.data_ptr(), a.data_ptr(), None, None, a.data_ptr(), 4, 4, 12, 12, 12, 4, 0, 2, 2, 0, None, 0, None, 0, stream())
    assert rc == -2 and b"multiples of 8" in lib.b200_last_error()


# ------------------------------------------------------------------ conv
@pytest.mark.parametrize("N,C,H,O,k,s,p,res,relu", [
    (2, 8, 56, 64, 7, 2, 3, False, True),     # stem after channel padding 3 -> 8
    (3, 8, 224, 64, 7, 2, 3, False, True),    # full-size stem: several output rows per CTA, image borders inside a CTA's rows
    (20, 8, 64, 48, 7, 2, 3, False, False),   # stem with fewer than 64 output channels, no ReLU
    (1, 64, 56, 64, 3, 1, 1, True, True),
    (2, 64, 56, 128, 3, 2, 1, False, True),
    (2, 64, 56, 128, 1, 2, 0, False, False),
    (3, 256, 14, 1024, 1, 1, 0, True, True),
    (1, 512, 7, 512, 3, 1, 1, False, True),
    (8, 64, 56, 64, 3, 1, 1, True, True),      # enough tiles for the persistent kernel, tiles cross image borders
    (32, 64, 56, 128, 3, 2, 1, False, True),   # persistent, stride 2
    (5, 128, 28, 128, 3, 1, 1, False, False),  # odd image count: the last tile runs past the tensor
    (16, 64, 56, 64, 3, 1, 1, False, True),    # several tiles per CTA: the 72 KB weight tile stays resident in shared memory
    (16, 64, 56, 512, 1, 1, 0, True, True),    # resident weights, two 256-wide column tiles: the weight tile is replaced mid-kernel
    (16, 128, 28, 256, 1, 1, 0, True, True),   # 128-wide tiles, two column tiles, residual
    (52, 256, 28, 64, 1, 1, 0, False, False),  # resident weights with four k-blocks per tile, ragged last tile
    (41, 128, 28, 512, 1, 1, 0, True, True),   # column tiles fastest: each CTA keeps one of four column tiles, ragged last row tile
    (37, 256, 14, 1024, 1, 1, 0, True, False), # column tiles fastest with eight column tiles (grid trimmed to a multiple of 8)
])
def test_conv2d_nhwc(lib, N, C, H, O, k, s, p, res, relu):
    dtype = torch.float16
    x = gen((N, C, H, H), dtype)
    w = gen((O, C, k, k), torch.float32, 1, math.sqrt(2.0 / (C * k * k)))
    gamma, beta = torch.rand(O) + 0.5, torch.randn(O) * 0.1
    mean, var = torch.randn(O) * 0.1, torch.rand(O) + 0.5
    Ho = (H + 2 * p - k) // s + 1
    r = gen((N, O, Ho, Ho), dtype, 5) if res else None
    ref = torch.nn.functional.conv2d(x.float(), w, None, s, p)
    ref = torch.nn.functional.batch_norm(ref, mean, var, gamma, beta, False, 0.0, 1e-5)
    if res:
        ref = ref + r.float()
    if relu:
        ref = torch.relu(ref)
    xd = x.cuda().contiguous(memory_format=torch.channels_last)
    wd = torch.empty(O * k * k * C, dtype=dtype, device="cuda")
    bd = torch.empty(O, dtype=torch.float32, device="cuda")
    prm = [t.cuda() for t in (gamma, beta, mean, var)]
    wc = w.cuda()
    ok(lib, lib.b200_conv_weight_prep(wc.data_ptr(), None, *[t.data_ptr() for t in prm], wd.data_ptr(), bd.data_ptr(), O, C, k, k, C,
                                      1e-5, 0, 0, 1, stream()))
    y = torch.empty(N, O, Ho, Ho, dtype=dtype, device="cuda").contiguous(memory_format=torch.channels_last)
    rd = r.cuda().contiguous(memory_format=torch.channels_last) if res else None
    ok(lib, lib.b200_conv2d_nhwc(xd.data_ptr(), wd.data_ptr(), bd.data_ptr(), rd.data_ptr() if res else None, y.data_ptr(), N, H, H, C, C,
                                 O, k, k, s, s, p, p, Ho, Ho, 1, 1 if relu else 0, stream()))
    close(y, ref, rtol=2e-2, atol=3e-2)


# ------------------------------------------------------------------ attention
def attn_ref(q, k, v, mask, scale, dtype):
    G = q.shape[1] // k.shape[1]
    k, v = k.float().repeat_interleave(G, 1), v.float().repeat_interleave(G, 1)
    s = q.float() @ k.transpose(-1, -2) * scale
    if mask is not None:
        s = s + mask.float()
    return torch.softmax(s, -1) @ v


@pytest.mark.parametrize("B,S,valid", [(1, 4352, 4097), (8, 4352, 4100), (3, 80, 37), (2, 272, 272), (64, 512, 300), (64, 4352, 4097), (5, 8192, 6000)])
def test_attn_decode(lib, B, S, valid):
    import model_zoo as mz

    dtype, Hq, Hkv, D = torch.bfloat16, 12, 2, 128
    q, k, v = gen((B, Hq, 1, D), dtype), gen((B, Hkv, S, D), dtype, 1), gen((B, Hkv, S, D), dtype, 2)
    mask = mz.causal_mask(B, 1, S, valid - 1)
    ref = attn_ref(q, k, v, mask, D ** -0.5, dtype)[:, :, 0]
    Q, K, V, M = q.cuda(), k.cuda(), v.cuda(), mask.cuda()
    out = torch.empty(B, Hq, D, dtype=dtype, device="cuda")
    ws = torch.empty(lib.b200_attn_decode_workspace_bytes(B, Hq, Hkv, S, D), dtype=torch.uint8, device="cuda")
    ok(lib, lib.b200_attn_decode(Q.data_ptr(), K.data_ptr(), V.data_ptr(), M.data_ptr(), out.data_ptr(), B, Hq, Hkv, S, D, Hq * D,
                                 Hkv * S * D, S * D, S, D ** -0.5, 2, ws.data_ptr(), ws.numel(), stream()))
    close(out, ref, rtol=2e-2, atol=5e-3)
    # no mask = attend to everything
    ok(lib, lib.b200_attn_decode(Q.data_ptr(), K.data_ptr(), V.data_ptr(), None, out.data_ptr(), B, Hq, Hkv, S, D, Hq * D,
                                 Hkv * S * D, S * D, 0, D ** -0.5, 2, ws.data_ptr(), ws.numel(), stream()))
    close(out, attn_ref(q, k, v, None, D ** -0.5, dtype)[:, :, 0], rtol=2e-2, atol=5e-3)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("B", [2, 12])
def test_attn_decode_small_batches_in_both_dtypes(lib, dtype, B):
    """Small batches take clusters of 16 splits (a non-portable cluster size that every kernel instantiation has to
    be allowed separately), B=12 the portable eight: both activation types, in one process, against the fp32 reference."""
    import model_zoo as mz

    S, valid, Hq, Hkv, D = 1024, 700, 12, 2, 128
    q, k, v = gen((B, Hq, 1, D), dtype), gen((B, Hkv, S, D), dtype, 1), gen((B, Hkv, S, D), dtype, 2)
    mask = mz.causal_mask(B, 1, S, valid - 1).to(dtype)
    ref = attn_ref(q, k, v, mask, D ** -0.5, dtype)[:, :, 0]
    Q, K, V, M = q.cuda(), k.cuda(), v.cuda(), mask.cuda()
    out = torch.empty(B, Hq, D, dtype=dtype, device="cuda")
    ws = torch.empty(max(16, lib.b200_attn_decode_workspace_bytes(B, Hq, Hkv, S, D)), dtype=torch.uint8, device="cuda")
    code = 2 if dtype == torch.bfloat16 else 1
    ok(lib, lib.b200_attn_decode(Q.data_ptr(), K.data_ptr(), V.data_ptr(), M.data_ptr(), out.data_ptr(), B, Hq, Hkv, S, D, Hq * D,
                                 Hkv * S * D, S * D, S, D ** -0.5, code, ws.data_ptr(), ws.numel(), stream()))
    close(out, ref, rtol=2e-2, atol=5e-3)


@pytest.mark.parametrize("B,S,Hq,Hkv", [(40, 2048, 12, 2), (64, 4352, 12, 2), (33, 1000, 8, 1), (130, 640, 4, 4)])
def test_attn_decode_many_sequences_ragged_masks(lib, B, S, Hq, Hkv):
    """Batches large enough for the balanced kernel (every CTA gets the same number of unmasked 16-key
    blocks): each sequence has its own attended length - from a single key to the whole cache - some
    masks have holes, and the call is repeated (the tickets of the merge must return to zero)."""
    dtype, D = torch.bfloat16, 128
    g = torch.Generator().manual_seed(B)
    q, k, v = gen((B, Hq, 1, D), dtype), gen((B, Hkv, S, D), dtype, 1), gen((B, Hkv, S, D), dtype, 2)
    neg = torch.finfo(dtype).min
    mask = torch.full((B, 1, 1, S), neg, dtype=dtype)
    lengths = torch.randint(1, S + 1, (B,), generator=g)
    lengths[0], lengths[1], lengths[2] = 1, S, 17
    for b in range(B):
        mask[b, 0, 0, :lengths[b]] = 0
        if b % 5 == 3 and lengths[b] > 200:      # a hole of masked keys inside the attended range
            mask[b, 0, 0, 64:160] = neg
        if b % 7 == 4:
            mask[b, 0, 0, :lengths[b]] = torch.where(torch.rand(int(lengths[b]), generator=g) < 0.5, 0.0, neg).to(dtype)
            mask[b, 0, 0, 0] = 0
    ref = attn_ref(q, k, v, mask, D ** -0.5, dtype)[:, :, 0]
    Q, K, V, M = q.cuda(), k.cuda(), v.cuda(), mask.cuda()
    ws = torch.empty(max(16, lib.b200_attn_decode_workspace_bytes(B, Hq, Hkv, S, D)), dtype=torch.uint8, device="cuda")
    for _ in range(2):
        out = torch.full((B, Hq, D), float("nan"), dtype=dtype, device="cuda")
        ok(lib, lib.b200_attn_decode(Q.data_ptr(), K.data_ptr(), V.data_ptr(), M.data_ptr(), out.data_ptr(), B, Hq, Hkv, S, D, Hq * D,
                                     Hkv * S * D, S * D, S, D ** -0.5, 2, ws.data_ptr(), ws.numel(), stream()))
        close(out, ref, rtol=2e-2, atol=5e-3)
    # a sequence whose mask admits no key gives zeros (ATen would average all rows; no model produces such a mask)
    mask[5] = neg
    out = torch.full((B, Hq, D), float("nan"), dtype=dtype, device="cuda")
    ok(lib, lib.b200_attn_decode(Q.data_ptr(), K.data_ptr(), V.data_ptr(), mask.cuda().data_ptr(), out.data_ptr(), B, Hq, Hkv, S, D, Hq * D,
                                 Hkv * S * D, S * D, S, D ** -0.5, 2, ws.data_ptr(), ws.numel(), stream()))
    assert (out[5] == 0).all()
    keep = [b for b in range(B) if b != 5]
    close(out[keep], ref[keep], rtol=2e-2, atol=5e-3)


@pytest.mark.parametrize("B,T", [(1, 512), (2, 48), (1, 100), (1, 2048), (2, 328)])
def test_attn_prefill(lib, B, T):
    import model_zoo as mz

    dtype, Hq, Hkv, D = torch.bfloat16, 12, 2, 128
    q = gen((B, T, Hq, D), dtype).transpose(1, 2)          # the layout the graph produces: a transposed view
    k, v = gen((B, Hkv, T, D), dtype, 1), gen((B, T, Hkv, D), dtype, 2).transpose(1, 2)
    mask = mz.causal_mask(1, T, T, 0)
    ref = attn_ref(q, k, v, mask, D ** -0.5, dtype).transpose(1, 2)
    Q, K, V, M = (t.cuda() for t in (q.transpose(1, 2).contiguous(), k, v.transpose(1, 2).contiguous(), mask))
    Q, V = Q.transpose(1, 2), V.transpose(1, 2)
    out = torch.full((B, T, Hq, D), float("nan"), dtype=dtype, device="cuda")
    st = lambda t: (C.c_int64 * 3)(*t.stride()[:3])
    ok(lib, lib.b200_attn_prefill(Q.data_ptr(), K.data_ptr(), V.data_ptr(), M.data_ptr(), out.data_ptr(), B, Hq, Hkv, T, T, D,
                                  st(Q), st(K), st(V), 0, T, D ** -0.5, 2, stream()))
    close(out, ref, rtol=2e-2, atol=5e-3)
    code = C.c_int(0)
    ok(lib, lib.b200_debug_device_error(C.byref(code), 1))
    assert code.value == 0


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_attn_prefill_arbitrary_masks_and_no_mask(lib, dtype):
    """Nothing in the kernels assumes a causal mask: a per-sequence mask with windows, holes and key
    tiles that are masked for a whole block of query rows (those tiles are skipped), S != T, and no
    mask at all."""
    B, T, S, Hq, Hkv, D = 2, 200, 456, 4, 2, 128
    g = torch.Generator().manual_seed(11)
    q, k, v = gen((B, Hq, T, D), dtype), gen((B, Hkv, S, D), dtype, 1), gen((B, Hkv, S, D), dtype, 2)
    neg = torch.finfo(dtype).min
    mask = torch.full((B, 1, T, S), neg, dtype=dtype)
    for b in range(B):
        for t in range(T):
            lo = (37 * t + 11 * b) % 300
            mask[b, 0, t, lo:lo + 40 + (t % 64)] = 0          # a sliding window; far tiles are fully masked
        mask[b, 0, :, 128:192] = neg                          # one key tile masked for every row
        mask[b, 0, :, 130 + b] = 0                            # ... except a single key
    mask[1, 0, 150:, 192:256] = torch.where(torch.rand(T - 150, 64, generator=g) < 0.3, 0.0, neg).to(dtype)
    ref = attn_ref(q, k, v, mask, D ** -0.5, dtype).transpose(1, 2)
    Q, K, V, M = q.cuda(), k.cuda(), v.cuda(), mask.cuda()
    out = torch.full((B, T, Hq, D), float("nan"), dtype=dtype, device="cuda")
    st = lambda t: (C.c_int64 * 3)(*t.stride()[:3])
    dt = DT[dtype]
    ok(lib, lib.b200_attn_prefill(Q.data_ptr(), K.data_ptr(), V.data_ptr(), M.data_ptr(), out.data_ptr(), B, Hq, Hkv, T, S, D,
                                  st(Q), st(K), st(V), T * S, S, D ** -0.5, dt, stream()))
    close(out, ref, rtol=2e-2, atol=5e-3)
    ok(lib, lib.b200_attn_prefill(Q.data_ptr(), K.data_ptr(), V.data_ptr(), None, out.data_ptr(), B, Hq, Hkv, T, S, D,
                                  st(Q), st(K), st(V), 0, 0, D ** -0.5, dt, stream()))
    close(out, attn_ref(q, k, v, None, D ** -0.5, dtype).transpose(1, 2), rtol=2e-2, atol=5e-3)
    code = C.c_int(0)
    ok(lib, lib.b200_debug_device_error(C.byref(code), 1))
    assert code.value == 0


# ------------------------------------------------------------------ bandwidth kernels
@pytest.mark.parametrize("rows,cols", [(1, 1536), (128, 1536), (2048, 1536), (5, 4096), (3, 100)])
def test_rmsnorm(lib, rows, cols):
    for dtype in (torch.bfloat16, torch.float16):
        x, w = gen((rows, cols), dtype), (1 + 0.02 * gen((cols,), torch.float32, 1)).to(dtype)
        n = (x.float() * torch.rsqrt(x.float().pow(2).mean(-1, keepdim=True) + 1e-6)).to(dtype)
        ref = (w.float() * n.float()).to(dtype)
        X, W = x.cuda(), w.cuda()
        Y = torch.empty_like(X)
        ok(lib, lib.b200_rmsnorm(X.data_ptr(), W.data_ptr(), Y.data_ptr(), rows, cols, cols, cols, 1e-6, DT[dtype], 1, stream()))
        got, r = Y.cpu(), ref
        ulp = (got.view(torch.int16).int() - r.view(torch.int16).int()).abs()
        # fp32 reduction order only: two roundings, so rarely 2 units in the last place
        assert ulp.max() <= 2 and (ulp != 0).float().mean() < 0.02 and (ulp > 1).float().mean() < 1e-4


@pytest.mark.parametrize("T", [1, 128, 1000, 2048])
def test_masked_softmax(lib, T):
    import model_zoo as mz

    dtype = torch.bfloat16
    H = 12 if T <= 1000 else 3
    x, mask = gen((1, H, T, T), dtype), mz.causal_mask(1, T, T, 0)
    ref = torch.softmax((x.float() + mask.float()).to(dtype).float(), -1)
    X, M = x.cuda(), mask.cuda()
    Y = torch.empty_like(X)
    ok(lib, lib.b200_softmax(X.data_ptr(), M.data_ptr(), Y.data_ptr(), 1, H, T, T, 0, 0, T, 1.0, 2, 2, 2, 1, stream()))
    close(Y, ref, rtol=1e-2, atol=2e-3)
    assert not Y.float().triu(1).any()            # masked positions are exactly zero
    Yf = torch.empty(1, H, T, T, dtype=torch.float32, device="cuda")
    ok(lib, lib.b200_softmax(X.data_ptr(), None, Yf.data_ptr(), 1, H, T, T, 0, 0, 0, 0.5, 2, 0, 0, 0, stream()))
    close(Yf, torch.softmax(x.float() * 0.5, -1), rtol=1e-3, atol=1e-5)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("T", [96, 2048, 8192])
def test_softmax_scale_and_finite_mask_round_like_the_unfused_ops(lib, T, dtype):
    """scale, then an additive mask of arbitrary finite values: each step rounds to the
    input dtype as the separate ATen ops would (the kernel may skip a rounding only where
    it cannot change the value)."""
    H, R = 2, 24
    code = 2 if dtype == torch.bfloat16 else 1
    x, mask = gen((1, H, R, T), dtype), gen((1, 1, R, T), dtype, 1)
    mask[..., ::3] = 0
    mask[..., 1::7] = float("-inf")
    scale = 128 ** -0.5
    ref = torch.softmax(((x.float() * scale).to(dtype).float() + mask.float()).to(dtype).float(), -1)
    X, M = x.cuda(), mask.cuda()
    Y = torch.empty_like(X)
    ok(lib, lib.b200_softmax(X.data_ptr(), M.data_ptr(), Y.data_ptr(), 1, H, R, T, 0, 0, T, scale, code, code, code, 1, stream()))
    close(Y, ref, rtol=1e-2, atol=1e-4)
    if dtype == torch.bfloat16:      # fp16 outputs can sit at the edge of underflow
        assert torch.equal(Y.cpu() == 0, ref.to(dtype) == 0)


def test_softmax_full_size_properties(lib):
    """[12, 8192, 8192] causal: too large for the CPU oracle in a test, so check what must
    hold: rows sum to 1, masked columns are 0, row 0 is one-hot."""
    T, H = 8192, 12
    x = torch.randn(1, H, T, T, device="cuda", dtype=torch.bfloat16, generator=torch.Generator("cuda").manual_seed(0))
    mask = torch.full((T, T), torch.finfo(torch.bfloat16).min, device="cuda", dtype=torch.bfloat16).triu(1)[None, None]
    y = torch.empty_like(x)
    ok(lib, lib.b200_softmax(x.data_ptr(), mask.data_ptr(), y.data_ptr(), 1, H, T, T, 0, 0, T, 1.0, 2, 2, 2, 1, stream()))
    for h in (0, H - 1):
        sums = y[0, h].float().sum(-1)
        assert (sums - 1).abs().max() < 2e-2
        assert not y[0, h].triu(1).any()
        assert y[0, h, 0, 0] == 1


@pytest.mark.parametrize("T", [1, 128, 2048])
def test_silu_mul_and_add_relu_chains(lib, T):
    from cuda_runtime import native

    dtype = torch.bfloat16
    g, u = gen((T, 8960), dtype), gen((T, 8960), dtype, 1)
    G, U = g.cuda(), u.cuda()
    Y = torch.empty_like(G)
    ins = (native.Tensor * 2)(bt(G), bt(U))
    ops = (native.EwOp * 2)(native.EwOp(2, 0, -1, 2, 0.0), native.EwOp(8, 4, 1, 2, 0.0))
    out = bt(Y)
    ok(lib, lib.b200_ew_chain(C.byref(out), ins, 2, ops, 2, stream()))
    ref = (torch.nn.functional.silu(g.float()).to(dtype).float() * u.float()).to(dtype)
    close(Y, ref, rtol=1e-2, atol=1e-2)
    ops = (native.EwOp * 2)(native.EwOp(7, 0, 1, 2, 0.0), native.EwOp(1, 4, -1, 2, 0.0))
    ok(lib, lib.b200_ew_chain(C.byref(out), ins, 2, ops, 2, stream()))
    assert torch.equal(Y.cpu(), torch.relu((g.float() + u.float()).to(dtype)))


def test_ew_chain_broadcast_and_strided(lib):
    from cuda_runtime import native

    x = gen((2, 5, 7, 16), torch.float16).cuda()
    b = gen((1, 5, 1, 1), torch.float32, 1).cuda()
    xt = x.permute(0, 2, 3, 1)                                  # channels-last style view
    y = torch.empty(2, 7, 16, 5, dtype=torch.float16, device="cuda")
    ins = (native.Tensor * 2)(bt(xt), bt(b.permute(0, 2, 3, 1).expand(2, 7, 16, 5)))
    ops = (native.EwOp * 3)(native.EwOp(8, 0, 1, 0, 0.0), native.EwOp(11, 4, -1, 0, 0.25), native.EwOp(3, 5, -1, 1, 0.0))
    out = bt(y)
    ok(lib, lib.b200_ew_chain(C.byref(out), ins, 2, ops, 3, stream()))
    ref = -(xt.float() * b.permute(0, 2, 3, 1) + 0.25)
    close(y, ref, rtol=2e-3, atol=2e-3)


@pytest.mark.parametrize("T", [1, 128, 2048])
def test_rope_table_and_rotate(lib, T):
    dtype, H, D = torch.bfloat16, 12, 128
    inv = 1.0 / (1e6 ** (torch.arange(0, D, 2).float() / D))
    pos = torch.arange(T) + 4096
    ang = torch.cat([pos.float()[:, None] * inv[None]] * 2, -1)
    cos, sin = ang.cos().to(dtype), ang.sin().to(dtype)
    INV, POS = inv.cuda(), pos.cuda()
    Cd, Sd = torch.empty(T, D, dtype=dtype, device="cuda"), torch.empty(T, D, dtype=dtype, device="cuda")
    ok(lib, lib.b200_rope_table(INV.data_ptr(), POS.data_ptr(), Cd.data_ptr(), Sd.data_ptr(), T, D, 4, 2, stream()))
    for got, ref in ((Cd, cos), (Sd, sin)):
        ulp = (got.cpu().view(torch.int16).int() - ref.view(torch.int16).int()).abs()
        assert ulp.max() <= 1 and (ulp != 0).float().mean() < 0.01
    x = gen((1, T, H, D), dtype).transpose(1, 2)
    xf = x.float()
    rot = torch.cat([-xf[..., D // 2:], xf[..., : D // 2]], -1)
    ref = ((xf * cos.float()).to(dtype).float() + (rot * sin.float()).to(dtype).float()).to(dtype)
    X = x.transpose(1, 2).contiguous().cuda().transpose(1, 2)
    Y = torch.empty(1, H, T, D, dtype=dtype, device="cuda")
    xs = bt(X)
    cos_d, sin_d = cos.cuda(), sin.cuda()
    ok(lib, lib.b200_rope_rotate(C.byref(xs), cos_d.data_ptr(), sin_d.data_ptr(), Y.data_ptr(), None, None, 0, 0, stream()))
    assert torch.equal(Y.cpu(), ref)


@pytest.mark.parametrize("M,N,K,fused", [(512, 1536, 8960, True), (1000, 1200, 4104, True), (300, 1536, 1024, False), (64, 1536, 8960, False)])
def test_linear_rmsnorm_equals_the_two_kernels(lib, M, N, K, fused):
    """b200_linear_rmsnorm = b200_linear then b200_rmsnorm.  On the CTA-pair split-K shapes the reduce kernel normalises the
    rows itself (the sum of squares is added in another order: last-bit differences); elsewhere the two kernels run as they are."""
    dtype = torch.bfloat16
    a, w, r = gen((M, K), dtype).cuda(), gen((N, K), dtype, 1, 0.05).cuda(), gen((M, N), dtype, 2).cuda()
    b, g = gen((N,), dtype, 3).cuda(), (1 + 0.1 * gen((N,), dtype, 4).float()).to(dtype).cuda()
    nb = lib.b200_linear_workspace_bytes(M, N, K)
    assert nb > 0 or not fused
    ws = torch.zeros(max(nb, 32), dtype=torch.uint8, device="cuda")
    h1, n1, h2, n2 = (torch.empty(M, N, dtype=dtype, device="cuda") for _ in range(4))
    for round_mid in (1, 0):
        ok(lib, lib.b200_linear_rmsnorm(a.data_ptr(), w.data_ptr(), b.data_ptr(), r.data_ptr(), h1.data_ptr(), M, N, K, K, K, N, N, 2, 2, 0,
                                        ws.data_ptr(), ws.numel(), g.data_ptr(), n1.data_ptr(), N, 1e-6, round_mid, stream()))
        ok(lib, lib.b200_linear(a.data_ptr(), w.data_ptr(), b.data_ptr(), r.data_ptr(), h2.data_ptr(), M, N, K, K, K, N, N, 2, 2, 0, None, 0,
                                ws.data_ptr(), ws.numel(), stream()))
        ok(lib, lib.b200_rmsnorm(h2.data_ptr(), g.data_ptr(), n2.data_ptr(), M, N, N, N, 1e-6, 2, round_mid, stream()))
        torch.cuda.synchronize()
        assert torch.equal(h1, h2)
        assert int(ws.count_nonzero()) == 0                     # the split-K workspace is left zeroed
        if fused:
            ulp = (n1.view(torch.int16).int() - n2.view(torch.int16).int()).abs()
            assert int(ulp.max()) <= 1 and float((ulp != 0).float().mean()) < 0.01
        else:
            assert torch.equal(n1, n2)
        hf = h2.float()
        x = hf * torch.rsqrt(hf.pow(2).mean(-1, keepdim=True) + 1e-6)
        if round_mid:
            x = x.to(dtype).float()
        close(n1, (x * g.float()).cpu(), rtol=2e-2, atol=2e-2)


@pytest.mark.parametrize("B,T", [(1, 512), (2, 37), (1, 5000)])
def test_rope_rotate_pair_equals_two_rotations(lib, B, T):
    """rope(q) and rope(k) of a prefill layer in one call, from column slices of the merged projection's
    output: bit-identical to two b200_rope_rotate calls (5000 positions: the two-launch form inside)."""
    dtype, Hq, Hkv, D = torch.bfloat16, 12, 2, 128
    N = (Hq + 2 * Hkv) * D
    qkv = gen((B, T, N), dtype).cuda()
    inv = 1.0 / (1e6 ** (torch.arange(0, D, 2).float() / D))
    ang = torch.cat([(torch.arange(T) + 3).float()[:, None] * inv[None]] * 2, -1)
    cos = ang.cos().to(dtype)[None].expand(B, T, D).contiguous().cuda()
    sin = ang.sin().to(dtype)[None].expand(B, T, D).contiguous().cuda()
    q = qkv[..., :Hq * D].view(B, T, Hq, D).transpose(1, 2)
    k = qkv[..., Hq * D:(Hq + Hkv) * D].view(B, T, Hkv, D).transpose(1, 2)
    qo, ko = torch.empty(B, Hq, T, D, dtype=dtype, device="cuda"), torch.empty(B, Hkv, T, D, dtype=dtype, device="cuda")
    qr, kr = torch.empty_like(qo), torch.empty_like(ko)
    qs, ks = bt(q), bt(k)
    ok(lib, lib.b200_rope_rotate_pair(C.byref(qs), C.byref(ks), cos.data_ptr(), sin.data_ptr(), qo.data_ptr(), ko.data_ptr(), stream()))
    ok(lib, lib.b200_rope_rotate(C.byref(qs), cos.data_ptr(), sin.data_ptr(), qr.data_ptr(), None, None, 0, 0, stream()))
    ok(lib, lib.b200_rope_rotate(C.byref(ks), cos.data_ptr(), sin.data_ptr(), kr.data_ptr(), None, None, 0, 0, stream()))
    assert torch.equal(qo, qr) and torch.equal(ko, kr)
    xf = k.float().cpu()
    rot = torch.cat([-xf[..., D // 2:], xf[..., : D // 2]], -1)
    c, s_ = cos.cpu().float()[:, None], sin.cpu().float()[:, None]
    assert torch.equal(ko.cpu(), ((xf * c).to(dtype).float() + (rot * s_).to(dtype).float()).to(dtype))
    # mismatched positions are refused
    k_bad = bt(k[:, :, : T - 1])
    assert lib.b200_rope_rotate_pair(C.byref(qs), C.byref(k_bad), cos.data_ptr(), sin.data_ptr(), qo.data_ptr(), ko.data_ptr(), stream()) == -1   # B200_EINVAL


@pytest.mark.parametrize("B,T", [(1, 1), (8, 1), (2, 5)])
def test_qkv_rope_cache_fused(lib, B, T):
    """rope(q), rope(k) -> key cache row, v -> value cache row in one launch, from column
    slices of one merged projection buffer (the layout the compiler produces)."""
    dtype, Hq, Hkv, D, S = torch.bfloat16, 12, 2, 128, 64
    N = (Hq + 2 * Hkv) * D
    qkv = gen((B, T, N), dtype)
    pos = torch.arange(T) + 17
    inv = 1.0 / (1e6 ** (torch.arange(0, D, 2).float() / D))
    ang = torch.cat([pos.float()[:, None] * inv[None]] * 2, -1)
    cos = ang.cos().to(dtype)[None].expand(B, T, D).contiguous()
    sin = ang.sin().to(dtype)[None].expand(B, T, D).contiguous()
    kc, vc = gen((B, Hkv, S, D), dtype, 1), gen((B, Hkv, S, D), dtype, 2)

    def heads(lo, n):  # [B,T,n*D] column slice -> [B,n,T,D] view
        return qkv[..., lo:lo + n * D].view(B, T, n, D).transpose(1, 2)

    def rope(x):
        xf = x.float()
        rot = torch.cat([-xf[..., D // 2:], xf[..., : D // 2]], -1)
        return ((xf * cos[:, None].float()).to(dtype).float() + (rot * sin[:, None].float()).to(dtype).float()).to(dtype)

    q, k, v = heads(0, Hq), heads(Hq * D, Hkv), heads((Hq + Hkv) * D, Hkv)
    ref_q = rope(q)
    ref_k, ref_v = kc.clone(), vc.clone()
    ref_k[:, :, pos] = rope(k)
    ref_v[:, :, pos] = v
    QKV, KC, VC, CO, SI, P = qkv.cuda(), kc.cuda(), vc.cuda(), cos.cuda(), sin.cuda(), pos.cuda()
    dv = lambda lo, n: QKV[..., lo:lo + n * D].view(B, T, n, D).transpose(1, 2)
    tq, tk, tv = bt(dv(0, Hq)), bt(dv(Hq * D, Hkv)), bt(dv((Hq + Hkv) * D, Hkv))
    qo = torch.empty(B, Hq, T, D, dtype=dtype, device="cuda")
    ok(lib, lib.b200_qkv_rope_cache(C.byref(tq), C.byref(tk), C.byref(tv), CO.data_ptr(), SI.data_ptr(), qo.data_ptr(), KC.data_ptr(),
                                    VC.data_ptr(), P.data_ptr(), S, 4, stream()))
    assert torch.equal(qo.cpu(), ref_q) and torch.equal(KC.cpu(), ref_k) and torch.equal(VC.cpu(), ref_v)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("B,norm,pos", [(1, True, 17), (8, True, 4100), (64, True, 4351), (5, False, -3), (64, False, 0)])
def test_linear_qkv_rope_equals_the_two_kernels(lib, dtype, B, norm, pos):
    """The merged q/k/v projection whose final pass rotates q and k and writes the cache rows is
    bit-identical to the projection followed by the rope / cache kernel - q, both caches whole."""
    Hq, Hkv, D, S, K = 12, 2, 128, 4352, 1536
    N = (Hq + 2 * Hkv) * D
    DTC = DT[dtype]
    x = gen((B, K), dtype, 0, 2.0).cuda()
    w, bias = gen((N, K), dtype, 1, 0.03).cuda(), gen((N,), dtype, 2).cuda()
    sumsq = x.float().pow(2).reshape(B, 24, K // 24).sum(-1).contiguous() if norm else None
    p_abs = pos if pos >= 0 else S + pos
    inv = 1.0 / (1e6 ** (torch.arange(0, D, 2).float() / D))
    ang = torch.cat([torch.full((B, 1), float(p_abs)) * inv[None]] * 2, -1)
    CO, SI = ang.cos().to(dtype).cuda().contiguous(), ang.sin().to(dtype).cuda().contiguous()
    kc0, vc0 = gen((B, Hkv, S, D), dtype, 3).cuda(), gen((B, Hkv, S, D), dtype, 4).cuda()
    P = torch.tensor([pos], dtype=torch.int64, device="cuda")
    sq_ptr, n_part = (sumsq.data_ptr(), 24) if norm else (None, 0)
    # two kernels
    qkv = torch.empty(B, N, dtype=dtype, device="cuda")
    ok(lib, lib.b200_linear_norm(x.data_ptr(), w.data_ptr(), bias.data_ptr(), None, qkv.data_ptr(), B, N, K, K, K, N, 0, DTC, DTC, 8,
                                 1e-6, sq_ptr, n_part, None, stream()))
    dv = lambda lo, n: qkv[:, None, lo:lo + n * D].view(B, 1, n, D).transpose(1, 2)
    tq, tk, tv = bt(dv(0, Hq)), bt(dv(Hq * D, Hkv)), bt(dv((Hq + Hkv) * D, Hkv))
    q_ref, k_ref, v_ref = torch.empty(B, Hq, 1, D, dtype=dtype, device="cuda"), kc0.clone(), vc0.clone()
    ok(lib, lib.b200_qkv_rope_cache(C.byref(tq), C.byref(tk), C.byref(tv), CO.data_ptr(), SI.data_ptr(), q_ref.data_ptr(), k_ref.data_ptr(),
                                    v_ref.data_ptr(), P.data_ptr(), S, 4, stream()))
    # one kernel
    q_out, kc, vc = torch.full((B, Hq, 1, D), float("nan"), dtype=dtype, device="cuda"), kc0.clone(), vc0.clone()
    ok(lib, lib.b200_linear_qkv_rope(x.data_ptr(), w.data_ptr(), bias.data_ptr(), B, N, K, K, K, DTC, DTC, 8, 1e-6, sq_ptr, n_part,
                                     CO.data_ptr(), SI.data_ptr(), q_out.data_ptr(), kc.data_ptr(), vc.data_ptr(), P.data_ptr(), S, 4, Hq, Hkv,
                                     stream()))
    torch.cuda.synchronize()
    as_bits = lambda t: t.cpu().view(torch.int16)
    assert torch.equal(as_bits(q_out), as_bits(q_ref))
    assert torch.equal(as_bits(kc), as_bits(k_ref)) and torch.equal(as_bits(vc), as_bits(v_ref))
    assert not torch.equal(as_bits(kc[:, :, p_abs]), as_bits(kc0[:, :, p_abs]))       # the row was written
    code = C.c_int(-1)
    ok(lib, lib.b200_debug_device_error(C.byref(code), 1))
    assert code.value == 0


def test_linear_qkv_rope_rejects_what_it_cannot_fuse(lib):
    x, w = gen((65, 1536), torch.bfloat16).cuda(), gen((2048, 1536), torch.bfloat16, 1).cuda()
    t = torch.zeros(65 * 12 * 128, dtype=torch.bfloat16, device="cuda")
    P = torch.zeros(1, dtype=torch.int64, device="cuda")
    args = lambda M, N, Hq: (x.data_ptr(), w.data_ptr(), None, M, N, 1536, 1536, 1536, 2, 2, 8, 0.0, None, 0, t.data_ptr(), t.data_ptr(),
                             t.data_ptr(), t.data_ptr(), t.data_ptr(), P.data_ptr(), 16, 4, Hq, 2, stream())
    assert lib.b200_linear_qkv_rope(*args(65, 2048, 12)) == -4      # more than 64 rows: B200_ENOTSUP
    assert lib.b200_linear_qkv_rope(*args(8, 2048, 10)) == -1       # N != (Hq + 2 Hkv) * 128: B200_EINVAL


def test_embedding_is_bit_exact(lib):
    V, D = 151936, 1536
    table = torch.randn(V, D, generator=torch.Generator().manual_seed(0)).bfloat16()
    ids = torch.tensor([0, V - 1, 70000, 65505, 2049, 151935, 1, 1], dtype=torch.int64)
    Tb, I = table.cuda(), ids.cuda()
    out = torch.empty(len(ids), D, dtype=torch.bfloat16, device="cuda")
    ok(lib, lib.b200_embedding(Tb.data_ptr(), I.data_ptr(), out.data_ptr(), len(ids), V, D * 2, 4, stream()))
    assert torch.equal(out.cpu().view(torch.int16), table[ids].view(torch.int16))
    I32 = ids.int().cuda()
    ok(lib, lib.b200_embedding(Tb.data_ptr(), I32.data_ptr(), out.data_ptr(), len(ids), V, D * 2, 3, stream()))
    assert torch.equal(out.cpu().view(torch.int16), table[ids].view(torch.int16))
    ok(lib, lib.b200_embedding(Tb.data_ptr(), I.data_ptr(), out.data_ptr(), 0, V, D * 2, 4, stream()))  # empty gather


@pytest.mark.parametrize("in_place", [True, False])
def test_index_copy_is_bit_exact(lib, in_place):
    B, H, S, D = 3, 2, 4352, 128
    cache, src = gen((B, H, S, D)), gen((B, 1, H, D), seed=1).transpose(1, 2)   # src is a strided view, as in the graph
    pos = torch.tensor([4100])
    ref = cache.index_copy(2, pos, src)
    Cc, Sc, P = cache.cuda(), src.transpose(1, 2).contiguous().cuda().transpose(1, 2), pos.cuda()
    dst = Cc if in_place else torch.zeros_like(Cc)
    ok(lib, lib.b200_index_copy(Cc.data_ptr(), dst.data_ptr(), Sc.data_ptr(), P.data_ptr(), B * H, S, D, 1, D, D * H, 2, 4, stream()))
    assert torch.equal(dst.cpu().view(torch.int16), ref.view(torch.int16))


def test_strided_copy_transpose_cast_and_pad(lib):
    x = gen((2, 3, 20, 20), torch.float32)
    X = x.cuda()
    full = torch.zeros(2, 20, 20, 8, dtype=torch.float16, device="cuda")
    dst = full.permute(0, 3, 1, 2)[:, :3]                       # NCHW-shaped window of an NHWC8 buffer
    a, b = bt(dst), bt(X)
    ok(lib, lib.b200_strided_copy(C.byref(a), C.byref(b), stream()))
    assert torch.equal(full[..., :3].cpu(), x.permute(0, 2, 3, 1).half()) and not full[..., 3:].any()
    y = gen((4, 6, 128), torch.bfloat16).cuda()
    z = torch.empty(6, 4, 128, dtype=torch.bfloat16, device="cuda")
    a, b = bt(z), bt(y.transpose(0, 1))
    ok(lib, lib.b200_strided_copy(C.byref(a), C.byref(b), stream()))
    assert torch.equal(z, y.transpose(0, 1).contiguous())


@pytest.mark.parametrize("N,Cn,H,W", [(3, 3, 5, 7), (2, 8, 4, 6), (1, 2, 33, 31)])
def test_strided_copy_planar_to_eight_channel_slots(lib, N, Cn, H, W):
    """Same-dtype NCHW -> NHWC8 window (the input repack of a convolution network): the
    channels of the window are replaced, the other channels of each slot keep their contents."""
    x = gen((N, Cn, H, W), torch.float16)
    X = x.cuda()
    full = torch.full((N, H, W, 8), 7.0, dtype=torch.float16, device="cuda")
    dst = full.permute(0, 3, 1, 2)[:, :Cn]
    a, b = bt(dst), bt(X)
    ok(lib, lib.b200_strided_copy(C.byref(a), C.byref(b), stream()))
    assert torch.equal(full[..., :Cn].cpu(), x.permute(0, 2, 3, 1))
    assert bool((full[..., Cn:] == 7.0).all())


def test_pooling_and_batchnorm(lib):
    x = gen((2, 64, 112, 112), torch.float16)
    for cl in (True, False):
        X = x.cuda().contiguous(memory_format=torch.channels_last) if cl else x.cuda()
        Y = torch.empty(2, 64, 56, 56, dtype=torch.float16, device="cuda")
        Y = Y.contiguous(memory_format=torch.channels_last) if cl else Y
        a, b = bt(X), bt(Y)
        ok(lib, lib.b200_max_pool2d(C.byref(a), C.byref(b), 3, 3, 2, 2, 1, 1, stream()))
        assert torch.equal(Y.cpu(), torch.nn.functional.max_pool2d(x.float(), 3, 2, 1).half())
        Z = torch.empty(2, 64, 1, 1, dtype=torch.float16, device="cuda")
        c = bt(Z)
        ok(lib, lib.b200_adaptive_avg_pool2d(C.byref(a), C.byref(c), stream()))
        close(Z, x.float().mean((2, 3), keepdim=True), rtol=2e-3, atol=2e-3)
    g, be, m, v = (torch.rand(64) + 0.5).cuda(), torch.randn(64).cuda(), torch.randn(64).cuda(), (torch.rand(64) + 0.5).cuda()
    X = x.cuda()
    Y = torch.empty_like(X)
    a, b = bt(X), bt(Y)
    ok(lib, lib.b200_batch_norm(C.byref(a), C.byref(b), g.data_ptr(), be.data_ptr(), m.data_ptr(), v.data_ptr(), 1e-5, 0, 0, stream()))
    close(Y, torch.nn.functional.batch_norm(x.float(), m.cpu(), v.cpu(), g.cpu(), be.cpu(), False, 0.0, 1e-5), rtol=2e-3, atol=4e-3)


def test_matmul_strided_and_mean_and_fill(lib):
    a, b = gen((2, 3, 20, 24), torch.bfloat16), gen((2, 1, 17, 24), torch.bfloat16, 1)
    A, B = a.cuda(), b.cuda()
    Bt = B.transpose(2, 3).expand(2, 3, 24, 17)
    out = torch.empty(2, 3, 20, 17, dtype=torch.bfloat16, device="cuda")
    arr = lambda t: (C.c_int64 * 4)(*t.stride())
    ok(lib, lib.b200_matmul_strided(A.data_ptr(), Bt.data_ptr(), out.data_ptr(), 2, 3, 20, 17, 24, arr(A), arr(Bt), arr(out), 2, stream()))
    close(out, a.float() @ b.float().transpose(2, 3), rtol=1e-2, atol=5e-2)
    x = gen((50, 333), torch.float32).cuda()
    y = torch.empty(50, dtype=torch.float32, device="cuda")
    ok(lib, lib.b200_mean_last_dim(x.data_ptr(), y.data_ptr(), 50, 333, 0, 0, stream()))
    close(y, x.mean(-1), rtol=1e-5, atol=1e-6)
    z = torch.empty(1000, dtype=torch.bfloat16, device="cuda")
    ok(lib, lib.b200_fill(z.data_ptr(), 1000, -2.5, 2, stream()))
    assert (z == -2.5).all()


def test_argmax_rows_matches_and_breaks_ties_low(lib):
    x = gen((9, 151936), torch.bfloat16)
    x[3, 77] = x[3, 150000] = 50.0
    X = x.cuda()
    out = torch.empty(9, dtype=torch.int64, device="cuda")
    ok(lib, lib.b200_argmax_rows(X.data_ptr(), out.data_ptr(), 9, 151936, 151936, 2, stream()))
    ref = torch.tensor([int(np.flatnonzero(r == r.max())[0]) for r in x.float().numpy()])
    assert torch.equal(out.cpu(), ref) and out[3] == 77
