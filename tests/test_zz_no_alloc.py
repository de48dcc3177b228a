"""The allocation-free decode attention entry point.

Some callers of the library cannot allocate device memory - a host runtime that has
already claimed the whole GPU, glue code that is only allowed to forward the pointers it
received.  ``b200_attn_decode_noalloc`` serves them from a scratch array built into the
library.  It must give what ``b200_attn_decode`` gives with a caller-provided workspace,
on the first call and on the next one (the array keeps the previous call's contents).
Collected last so that a run which stops at the first failure has already run everything else.
"""

import pytest
import torch

pytestmark = pytest.mark.gpu


def _case(B, S, valid, seed):
    import model_zoo as mz

    g = torch.Generator().manual_seed(seed)
    Hq, Hkv, D = 12, 2, 128
    q = torch.randn(B, Hq, D, generator=g).bfloat16().cuda()
    k = torch.randn(B, Hkv, S, D, generator=g).bfloat16().cuda()
    v = torch.randn(B, Hkv, S, D, generator=g).bfloat16().cuda()
    mask = mz.causal_mask(B, 1, S, valid - 1).reshape(B, S).cuda()
    return q, k, v, mask, Hq, Hkv, D


def _attn_ref(q, k, v, mask, scale):
    """fp32 statement of the op on the host: softmax(q k^T * scale + mask) v with shared KV heads."""
    G = q.shape[1] // k.shape[1]
    kf, vf = k.float().cpu().repeat_interleave(G, 1), v.float().cpu().repeat_interleave(G, 1)
    s = torch.einsum("bhd,bhsd->bhs", q.float().cpu(), kf) * scale + mask.float().cpu()[:, None, :]
    return torch.einsum("bhs,bhsd->bhd", torch.softmax(s, -1), vf)


def _run_pair(lib, B, S, valid, seed):
    stream = torch.cuda.current_stream().cuda_stream
    q, k, v, mask, Hq, Hkv, D = _case(B, S, valid, seed)
    scale = D ** -0.5
    need = lib.b200_attn_decode_workspace_bytes(B, Hq, Hkv, S, D)
    ws = torch.empty(max(need, 16), dtype=torch.uint8, device="cuda")
    want = torch.empty(B, Hq, D, dtype=torch.bfloat16, device="cuda")
    got = torch.full_like(want, float("nan"))
    rc = lib.b200_attn_decode(q.data_ptr(), k.data_ptr(), v.data_ptr(), mask.data_ptr(), want.data_ptr(), B, Hq, Hkv, S, D, Hq * D,
                              Hkv * S * D, S * D, S, scale, 2, ws.data_ptr(), ws.numel(), stream)
    assert rc == 0, lib.b200_last_error().decode()
    rc = lib.b200_attn_decode_noalloc(q.data_ptr(), k.data_ptr(), v.data_ptr(), mask.data_ptr(), got.data_ptr(), B, Hq, Hkv, S, D,
                                      Hq * D, Hkv * S * D, S * D, S, scale, 2, stream)
    assert rc == 0, lib.b200_last_error().decode()
    torch.cuda.synchronize()
    torch.testing.assert_close(got.float(), want.float(), rtol=2e-2, atol=5e-3)
    torch.testing.assert_close(got.float().cpu(), _attn_ref(q, k, v, mask, scale), rtol=2e-2, atol=5e-3)
    return need


def test_noalloc_uses_the_builtin_scratch_twice_in_a_row(native_lib):
    """Shapes whose split-KV partials go through global scratch (caches longer than the in-kernel
    merge covers, or too short for it): the built-in array is what the kernels read and write.  Two
    calls in a row with different layouts of the partials - the second finds the first one's data
    in the array - must both equal the workspace entry point and the fp32 host statement."""
    lib = native_lib
    torch.cuda.set_device(0)
    for B, S, valid, seed in ((2, 20000, 19000, 0), (3, 24000, 5000, 1), (3, 80, 37, 2)):
        need = _run_pair(lib, B, S, valid, seed)
        assert 0 < need <= 8 << 20, f"B={B} S={S} no longer plans to the scratch path (needs {need} bytes)"


def test_noalloc_shapes_that_need_no_scratch(native_lib):
    """Caches of 512..16384 rows merge their splits inside the kernel; the entry point must serve them too."""
    lib = native_lib
    torch.cuda.set_device(0)
    for B, S, valid, seed in ((8, 4352, 4100, 0), (3, 1024, 700, 1), (8, 6144, 6000, 2)):
        _run_pair(lib, B, S, valid, seed)


def test_noalloc_rejects_shapes_beyond_the_builtin_scratch(native_lib):
    lib = native_lib
    # 2000 sequences over a 32768-row cache: the per-split partials (~800 MB) do not fit the 8 MiB array.
    B, S = 2000, 32768
    assert lib.b200_attn_decode_workspace_bytes(B, 12, 2, S, 128) > 8 << 20
    dummy = torch.zeros(16, dtype=torch.bfloat16, device="cuda")
    rc = lib.b200_attn_decode_noalloc(dummy.data_ptr(), dummy.data_ptr(), dummy.data_ptr(), None, dummy.data_ptr(), B, 12, 2, S, 128,
                                      12 * 128, 2 * S * 128, S * 128, 0, 0.088, 2, torch.cuda.current_stream().cuda_stream)
    assert rc == -5 and b"built-in array" in lib.b200_last_error()
