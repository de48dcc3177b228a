"""Host stand-in for ``libb200nn.so`` - TEST INFRASTRUCTURE ONLY.

The CPU test-suite installs this object through
``cuda_runtime.native.install_test_library`` so that the whole host pipeline
(IR -> patterns -> lowering -> arena plan -> argument binding -> outputs) can be
checked against the oracle on a machine without a GPU.  Every method has the
argument list of the C entry point of the same name (include/b200nn.h) and
computes the documented result with plain torch ops on the raw host addresses it
is given.  It proves nothing about the CUDA kernels; the ``gpu`` tests do that.
"""

from __future__ import annotations

import ctypes as C
import math

import torch

_DT = {0: torch.float32, 1: torch.float16, 2: torch.bfloat16, 3: torch.int32, 4: torch.int64, 5: torch.uint8}
_MAX_IN = 4
_OPS = ("RELU", "SILU", "NEG", "RSQRT", "COS", "SIN", "ADD", "MUL", "DIV", "SUB", "ADD_S", "MUL_S", "DIV_S", "POW_S", "SUB_S",
        "CAST", "SIGMOID", "EXP", "SQRT", "TANH", "GELU", "RSUB_S", "MAX", "MIN")


def _addr(p):
    if p is None:
        return None
    if isinstance(p, int):
        return p
    if hasattr(p, "_obj"):
        return p._obj
    if hasattr(p, "value"):
        return p.value
    return p


def _raw(ptr, dtype, shape, strides):
    """torch view over host memory at ``ptr``."""
    ptr = _addr(ptr)
    shape = [int(s) for s in shape]
    strides = [int(s) for s in strides]
    if any(s == 0 for s in shape):
        return torch.empty(shape, dtype=dtype)
    extent = 1 + sum((s - 1) * st for s, st in zip(shape, strides))
    item = torch.empty(0, dtype=dtype).element_size()
    buf = (C.c_char * (extent * item)).from_address(ptr)
    return torch.frombuffer(buf, dtype=dtype, count=extent).as_strided(shape, strides)


def _flat(ptr, dtype_code, n):
    return _raw(ptr, _DT[dtype_code], [n], [1])


def _t(struct):
    s = _addr(struct)
    nd = s.ndim
    return _raw(s.data, _DT[s.dtype], list(s.shape)[:nd], list(s.stride)[:nd])


def _round(x, code):
    return x.to(_DT[code]).float() if code in (1, 2) else x


class FakeLibrary:
    def __init__(self):
        self.calls: list[str] = []
        self._err = b""

    # -- misc ---------------------------------------------------------------
    def b200_version(self):
        return 1

    def b200_last_error(self):
        return self._err

    def b200_debug_wait_timeout(self, probes, stream):
        return 0

    def b200_linear_workspace_bytes(self, M, N, K):
        return 256 if M <= 128 else 0

    def b200_attn_decode_workspace_bytes(self, B, Hq, Hkv, S, D):
        return 256

    # -- elementwise ------------------------------------------------------------
    def b200_ew_chain(self, out, ins, n_in, ops, n_ops, stream):
        self.calls.append("ew_chain")
        o = _t(out)
        slots = {i: _t(ins[i]).float() for i in range(n_in)}
        r = None
        for j in range(n_ops):
            op = ops[j]
            name = _OPS[op.opcode - 1]
            a = slots[op.a]
            b = slots[op.b] if op.b >= 0 else None
            imm = op.imm
            if name == "RELU": r = torch.relu(a)
            elif name == "SILU": r = a / (1 + torch.exp(-a))
            elif name == "NEG": r = -a
            elif name == "RSQRT": r = torch.rsqrt(a)
            elif name == "COS": r = torch.cos(a)
            elif name == "SIN": r = torch.sin(a)
            elif name == "ADD": r = a + b
            elif name == "MUL": r = a * b
            elif name == "DIV": r = a / b
            elif name == "SUB": r = a - b
            elif name == "ADD_S": r = a + imm
            elif name == "MUL_S": r = a * imm
            elif name == "DIV_S": r = a / imm
            elif name == "POW_S": r = a ** imm
            elif name == "SUB_S": r = a - imm
            elif name == "RSUB_S": r = imm - a
            elif name == "CAST": r = a
            elif name == "SIGMOID": r = torch.sigmoid(a)
            elif name == "EXP": r = torch.exp(a)
            elif name == "SQRT": r = torch.sqrt(a)
            elif name == "TANH": r = torch.tanh(a)
            elif name == "GELU": r = torch.nn.functional.gelu(a)
            elif name == "MAX": r = torch.maximum(a, b)
            elif name == "MIN": r = torch.minimum(a, b)
            r = _round(r, op.round_dtype)
            slots[_MAX_IN + j] = r
        o.copy_(r.to(o.dtype))
        return 0

    def b200_strided_copy(self, out, inp, stream):
        self.calls.append("strided_copy")
        o, i = _t(out), _t(inp)
        o.copy_(i.to(o.dtype))
        return 0

    def b200_fill(self, out, n, value, dtype, stream):
        self.calls.append("fill")
        _flat(out, dtype, n).fill_(value)
        return 0

    # -- reductions ----------------------------------------------------------------
    def b200_rmsnorm(self, x, w, y, rows, cols, xs, ys, eps, dtype, round_mid, stream):
        self.calls.append("rmsnorm")
        dt = _DT[dtype]
        X = _raw(x, dt, [rows, cols], [xs, 1]).float()
        W = _raw(w, dt, [cols], [1]).float()
        n = X * torch.rsqrt(X.pow(2).mean(-1, keepdim=True) + eps)
        if round_mid:
            n = n.to(dt).float()
        _raw(y, dt, [rows, cols], [ys, 1]).copy_((n * W).to(dt))
        return 0

    def b200_softmax(self, x, mask, y, d0, d1, d2, cols, ms0, ms1, ms2, scale, in_dtype, mask_dtype, out_dtype, round_steps, stream):
        self.calls.append("softmax")
        dt = _DT[in_dtype]
        shape = [d0, d1, d2, cols]
        cs = [d1 * d2 * cols, d2 * cols, cols, 1]
        t = _raw(x, dt, shape, cs).float()
        if scale != 1.0:
            t = t * scale
            if round_steps:
                t = t.to(dt).float()
        if _addr(mask):
            t = t + _raw(mask, _DT[mask_dtype], shape, [ms0, ms1, ms2, 1]).float()
            if round_steps:
                t = t.to(dt).float()
        _raw(y, _DT[out_dtype], shape, cs).copy_(torch.softmax(t, -1).to(_DT[out_dtype]))
        return 0

    def b200_mean_last_dim(self, x, y, rows, cols, in_dtype, out_dtype, stream):
        self.calls.append("mean_last_dim")
        X = _raw(x, _DT[in_dtype], [rows, cols], [cols, 1]).float()
        _flat(y, out_dtype, rows).copy_(X.mean(-1).to(_DT[out_dtype]))
        return 0

    def b200_argmax_rows(self, x, out, rows, cols, row_stride, dtype, stream):
        self.calls.append("argmax")
        X = _raw(x, _DT[dtype], [rows, cols], [row_stride, 1]).float()
        _flat(out, 4, rows).copy_(X.argmax(-1))
        return 0

    # -- indexing ---------------------------------------------------------------------
    def b200_embedding(self, table, ids, out, n_ids, vocab, row_bytes, ids_dtype, stream):
        self.calls.append("embedding")
        T = _raw(table, torch.uint8, [vocab, row_bytes], [row_bytes, 1])
        I = _flat(ids, ids_dtype, n_ids).long()
        _raw(out, torch.uint8, [n_ids, row_bytes], [row_bytes, 1]).copy_(T[I])
        return 0

    def b200_index_copy(self, base, dst, src, index, outer, dim_size, inner, n_index, so, si, elem_bytes, index_dtype, stream):
        self.calls.append("index_copy")
        ib = inner * elem_bytes
        D = _raw(dst, torch.uint8, [outer, dim_size, ib], [dim_size * ib, ib, 1])
        if _addr(base) != _addr(dst):
            D.copy_(_raw(base, torch.uint8, [outer, dim_size, ib], [dim_size * ib, ib, 1]))
        S = _raw(src, torch.uint8, [outer, n_index, ib], [so * elem_bytes, si * elem_bytes, 1])
        I = _flat(index, index_dtype, n_index).long()
        D[:, I, :] = S
        return 0

    def b200_rope_table(self, inv_freq, positions, cos_out, sin_out, n_pos, head_dim, pos_dtype, out_dtype, stream):
        self.calls.append("rope_table")
        inv = _flat(inv_freq, 0, head_dim // 2)
        pos = _flat(positions, pos_dtype, n_pos).float()
        ang = pos[:, None] * inv[None, :]
        ang = torch.cat([ang, ang], -1)
        _raw(cos_out, _DT[out_dtype], [n_pos, head_dim], [head_dim, 1]).copy_(ang.cos().to(_DT[out_dtype]))
        _raw(sin_out, _DT[out_dtype], [n_pos, head_dim], [head_dim, 1]).copy_(ang.sin().to(_DT[out_dtype]))
        return 0

    def b200_rope_rotate(self, x, cos_t, sin_t, y, kv_cache, cache_pos, cache_len, pos_dtype, stream):
        self.calls.append("rope_rotate")
        X = _t(x)
        dt = X.dtype
        B, H, T, D = X.shape
        c = _raw(cos_t, dt, [B, 1, T, D], [T * D, T * D, D, 1]).float()
        s = _raw(sin_t, dt, [B, 1, T, D], [T * D, T * D, D, 1]).float()
        xf = X.float()
        rot = torch.cat([-xf[..., D // 2:], xf[..., :D // 2]], -1)
        r = ((xf * c).to(dt).float() + (rot * s).to(dt).float()).to(dt)
        _raw(y, dt, [B, H, T, D], [H * T * D, T * D, D, 1]).copy_(r)
        return 0

    def b200_rope_rotate_pair(self, q, k, cos_t, sin_t, q_out, k_out, stream):
        self.b200_rope_rotate(q, cos_t, sin_t, q_out, None, None, 0, 0, stream)
        self.b200_rope_rotate(k, cos_t, sin_t, k_out, None, None, 0, 0, stream)
        self.calls[-2:] = ["rope_rotate_pair"]
        return 0

    def b200_qkv_rope_cache(self, q, k, v, cos_t, sin_t, q_out, k_cache, v_cache, cache_pos, cache_len, pos_dtype, stream):
        self.calls.append("qkv_rope_cache")
        Q, K, Vv = _t(q), _t(k), _t(v)
        dt = Q.dtype
        B, Hq, T, D = Q.shape
        Hkv = K.shape[1]
        c = _raw(cos_t, dt, [B, 1, T, D], [T * D, T * D, D, 1]).float()
        s = _raw(sin_t, dt, [B, 1, T, D], [T * D, T * D, D, 1]).float()

        def rope(x):
            xf = x.float()
            rot = torch.cat([-xf[..., D // 2:], xf[..., :D // 2]], -1)
            return ((xf * c).to(dt).float() + (rot * s).to(dt).float()).to(dt)

        _raw(q_out, dt, [B, Hq, T, D], [Hq * T * D, T * D, D, 1]).copy_(rope(Q))
        pos = _flat(cache_pos, pos_dtype, T).long()
        cs = [Hkv * cache_len * D, cache_len * D, D, 1]
        _raw(k_cache, dt, [B, Hkv, cache_len, D], cs)[:, :, pos] = rope(K)
        _raw(v_cache, dt, [B, Hkv, cache_len, D], cs)[:, :, pos] = Vv
        return 0

    # -- CNN ops --------------------------------------------------------------------
    def b200_max_pool2d(self, x, y, kh, kw, sh, sw, ph, pw, stream):
        self.calls.append("max_pool2d")
        X, Y = _t(x), _t(y)
        Y.copy_(torch.nn.functional.max_pool2d(X.float(), (kh, kw), (sh, sw), (ph, pw)).to(Y.dtype))
        return 0

    def b200_adaptive_avg_pool2d(self, x, y, stream):
        self.calls.append("adaptive_avg_pool2d")
        X, Y = _t(x), _t(y)
        Y.copy_(torch.nn.functional.adaptive_avg_pool2d(X.float(), Y.shape[2:]).to(Y.dtype))
        return 0

    def b200_batch_norm(self, x, y, gamma, beta, mean, var, eps, param_dtype, relu, stream):
        self.calls.append("batch_norm")
        X, Y = _t(x), _t(y)
        Cn = X.shape[1]
        g = lambda p, d: _flat(p, param_dtype, Cn).float() if _addr(p) else torch.full((Cn,), d)
        r = torch.nn.functional.batch_norm(X.float(), g(mean, 0.0), g(var, 1.0), g(gamma, 1.0), g(beta, 0.0), False, 0.0, eps)
        Y.copy_((torch.relu(r) if relu else r).to(Y.dtype))
        return 0

    def b200_conv_weight_prep(self, w, conv_bias, gamma, beta, mean, var, w_out, bias_out, O, I, KH, KW, I_pad, eps, w_dtype,
                              param_dtype, out_dtype, stream):
        self.calls.append("conv_weight_prep")
        Wt = _raw(w, _DT[w_dtype], [O, I, KH, KW], [I * KH * KW, KH * KW, KW, 1]).float()
        vec = lambda p, d: _flat(p, param_dtype, O).float() if _addr(p) else torch.full((O,), d)
        b = vec(conv_bias, 0.0)
        if _addr(var):
            scale = vec(gamma, 1.0) / torch.sqrt(vec(var, 1.0) + eps)
            b = vec(beta, 0.0) + (b - vec(mean, 0.0)) * scale
            Wt = Wt * scale[:, None, None, None]
        packed = torch.zeros(O, KH, KW, I_pad)
        packed[..., :I] = Wt.permute(0, 2, 3, 1)
        _flat(w_out, out_dtype, O * KH * KW * I_pad).copy_(packed.reshape(-1).to(_DT[out_dtype]))
        _flat(bias_out, 0, O).copy_(b)
        return 0

    # -- contractions ------------------------------------------------------------------
    def b200_linear(self, A, W, bias, residual, out, M, N, K, lda, ldw, ldo, ldr, dtype, bias_dtype, epilogue, aux, ldaux,
                    workspace, workspace_bytes, stream):
        self.calls.append("linear")
        dt = _DT[dtype]
        a = _raw(A, dt, [M, K], [lda, 1]).float()
        w = _raw(W, dt, [N, K], [ldw, 1]).float()
        r = a @ w.t()
        if _addr(bias):
            r = r + _flat(bias, bias_dtype, N).float()
        if epilogue & 4:  # gated MLP: gate/up rows interleaved in blocks of 64
            r = r.reshape(M, N // 128, 2, 64)
            g, u = r[:, :, 0].to(dt).float(), r[:, :, 1].to(dt).float()
            r = ((g / (1 + torch.exp(-g))).to(dt).float() * u).reshape(M, N // 2)
            _raw(out, dt, [M, N // 2], [ldo, 1]).copy_(r.to(dt))
            return 0
        if _addr(residual):
            r = r.to(dt).float() + _raw(residual, dt, [M, N], [ldr, 1]).float()
        if epilogue & 1:
            r = torch.relu(r)
        if epilogue & 2:
            s = r.to(dt).float()
            r = (s / (1 + torch.exp(-s))).to(dt).float() * _raw(aux, dt, [M, N], [ldaux, 1]).float()
        _raw(out, dt, [M, N], [ldo, 1]).copy_(r.to(dt))
        return 0

    def b200_linear_rmsnorm(self, A, W, bias, residual, out, M, N, K, lda, ldw, ldo, ldr, dtype, bias_dtype, epilogue, workspace,
                            workspace_bytes, norm_weight, norm_out, ldn, norm_eps, round_mid, stream):
        self.b200_linear(A, W, bias, residual, out, M, N, K, lda, ldw, ldo, ldr, dtype, bias_dtype, epilogue, None, 0, workspace,
                         workspace_bytes, stream)
        self.b200_rmsnorm(out, norm_weight, norm_out, M, N, ldo, ldn, norm_eps, dtype, round_mid, stream)
        self.calls[-2:] = ["linear_rmsnorm"]
        return 0

    def b200_linear_norm(self, A, W, bias, residual, out, M, N, K, lda, ldw, ldo, ldr, dtype, bias_dtype, epilogue, norm_eps,
                         sumsq_in, sumsq_in_cols, sumsq_out, stream):
        self.calls.append("linear_norm")
        assert M <= 64
        dt = _DT[dtype]
        a = _raw(A, dt, [M, K], [lda, 1]).float()
        w = _raw(W, dt, [N, K], [ldw, 1]).float()
        r = a @ w.t()
        if _addr(sumsq_in):   # RMSNorm of the input rows applied after the GEMM (gain folded into W by the caller)
            assert 0 < sumsq_in_cols <= 32
            ss = _raw(sumsq_in, torch.float32, [M, sumsq_in_cols], [sumsq_in_cols, 1]).sum(-1, keepdim=True)
            r = r * torch.rsqrt(ss / K + norm_eps)
        if _addr(bias):
            r = r + _flat(bias, bias_dtype, N).float()
        if epilogue & 4:
            r = r.reshape(M, N // 128, 2, 64)
            g, u = r[:, :, 0].to(dt).float(), r[:, :, 1].to(dt).float()
            _raw(out, dt, [M, N // 2], [ldo, 1]).copy_(((g / (1 + torch.exp(-g))).to(dt).float() * u).reshape(M, N // 2).to(dt))
            return 0
        if _addr(residual):
            r = r.to(dt).float() + _raw(residual, dt, [M, N], [ldr, 1]).float()
        if epilogue & 1:
            r = torch.relu(r)
        r = r.to(dt)
        _raw(out, dt, [M, N], [ldo, 1]).copy_(r)
        if _addr(sumsq_out):
            assert N % 64 == 0
            _raw(sumsq_out, torch.float32, [M, N // 64], [N // 64, 1]).copy_(r.float().pow(2).reshape(M, N // 64, 64).sum(-1))
        return 0

    def b200_linear_qkv_rope(self, A, W, bias, M, N, K, lda, ldw, dtype, bias_dtype, epilogue, norm_eps, sumsq_in, sumsq_in_cols,
                             cos_t, sin_t, q_out, k_cache, v_cache, cache_pos, cache_len, pos_dtype, Hq, Hkv, stream):
        self.calls.append("linear_qkv_rope")
        assert M <= 64 and N == (Hq + 2 * Hkv) * 128 and not (epilogue & ~8)
        dt = _DT[dtype]
        D = 128
        r = _raw(A, dt, [M, K], [lda, 1]).float() @ _raw(W, dt, [N, K], [ldw, 1]).float().t()
        if _addr(sumsq_in):
            ss = _raw(sumsq_in, torch.float32, [M, sumsq_in_cols], [sumsq_in_cols, 1]).sum(-1, keepdim=True)
            r = r * torch.rsqrt(ss / K + norm_eps)
        if _addr(bias):
            r = r + _flat(bias, bias_dtype, N).float()
        r = r.to(dt).reshape(M, Hq + 2 * Hkv, D)
        c = _raw(cos_t, dt, [M, 1, D], [D, D, 1]).float()
        s = _raw(sin_t, dt, [M, 1, D], [D, D, 1]).float()

        def rope(x):
            xf = x.float()
            rot = torch.cat([-xf[..., D // 2:], xf[..., :D // 2]], -1)
            return ((xf * c).to(dt).float() + (rot * s).to(dt).float()).to(dt)

        _raw(q_out, dt, [M, Hq, D], [Hq * D, D, 1]).copy_(rope(r[:, :Hq]))
        pos = int(_flat(cache_pos, pos_dtype, 1)[0])
        pos = pos + cache_len if pos < 0 else pos
        if 0 <= pos < cache_len:
            cs = [Hkv * cache_len * D, cache_len * D, D, 1]
            _raw(k_cache, dt, [M, Hkv, cache_len, D], cs)[:, :, pos] = rope(r[:, Hq:Hq + Hkv])
            _raw(v_cache, dt, [M, Hkv, cache_len, D], cs)[:, :, pos] = r[:, Hq + Hkv:]
        return 0

    def b200_matmul_strided(self, A, B, out, b1, b2, M, N, K, a_s, b_s, o_s, dtype, stream):
        self.calls.append("matmul")
        dt = _DT[dtype]
        a = _raw(A, dt, [b1, b2, M, K], list(a_s)).float()
        b = _raw(B, dt, [b1, b2, K, N], list(b_s)).float()
        _raw(out, dt, [b1, b2, M, N], list(o_s)).copy_((a @ b).to(dt))
        return 0

    def b200_conv2d_nhwc(self, x, w, bias, residual, y, N, H, W, Cn, C_pad, O, KH, KW, sh, sw, ph, pw, Ho, Wo, dtype, epilogue,
                         stream):
        self.calls.append("conv2d")
        dt = _DT[dtype]
        X = _raw(x, dt, [N, Cn, H, W], [H * W * Cn, 1, W * Cn, Cn]).float()
        Wt = _raw(w, dt, [O, Cn, KH, KW], [KH * KW * Cn, 1, KW * Cn, Cn]).float()
        r = torch.nn.functional.conv2d(X, Wt, _flat(bias, 0, O) if _addr(bias) else None, (sh, sw), (ph, pw))
        nhwc = [Ho * Wo * O, 1, Wo * O, O]
        if _addr(residual):
            r = r + _raw(residual, dt, [N, O, Ho, Wo], nhwc).float()
        if epilogue & 1:
            r = torch.relu(r)
        _raw(y, dt, [N, O, Ho, Wo], nhwc).copy_(r.to(dt))
        return 0

    # -- attention ----------------------------------------------------------------------
    def _attn(self, q, k, v, mask, scale, dt):
        Hq, Hkv = q.shape[1], k.shape[1]
        k = k.repeat_interleave(Hq // Hkv, 1)
        v = v.repeat_interleave(Hq // Hkv, 1)
        s = q @ k.transpose(-1, -2) * scale
        if mask is not None:
            s = s + mask
        p = torch.softmax(s, -1).to(dt).float()
        return p @ v

    def b200_attn_decode(self, q, k, v, mask, out, B, Hq, Hkv, S, D, q_bs, kv_bs, kv_hs, mask_bs, scale, dtype, ws, ws_bytes, stream):
        self.calls.append("attn_decode")
        dt = _DT[dtype]
        Q = _raw(q, dt, [B, Hq, 1, D], [q_bs, D, D, 1]).float()
        K = _raw(k, dt, [B, Hkv, S, D], [kv_bs, kv_hs, D, 1]).float()
        Vv = _raw(v, dt, [B, Hkv, S, D], [kv_bs, kv_hs, D, 1]).float()
        M = _raw(mask, dt, [B, 1, 1, S], [mask_bs, 0, 0, 1]).float() if _addr(mask) else None
        o = self._attn(Q, K, Vv, M, scale, dt)
        _raw(out, dt, [B, Hq, D], [Hq * D, D, 1]).copy_(o[:, :, 0, :].to(dt))
        return 0

    def b200_attn_prefill(self, q, k, v, mask, out, B, Hq, Hkv, T, S, D, qs, ks, vs, mask_b, mask_t, scale, dtype, stream):
        self.calls.append("attn_prefill")
        dt = _DT[dtype]
        Q = _raw(q, dt, [B, Hq, T, D], list(qs)[:3] + [1]).float()
        K = _raw(k, dt, [B, Hkv, S, D], list(ks)[:3] + [1]).float()
        Vv = _raw(v, dt, [B, Hkv, S, D], list(vs)[:3] + [1]).float()
        M = _raw(mask, dt, [B, 1, T, S], [mask_b, 0, mask_t, 1]).float() if _addr(mask) else None
        o = self._attn(Q, K, Vv, M, scale, dt)
        _raw(out, dt, [B, T, Hq, D], [T * Hq * D, Hq * D, D, 1]).copy_(o.transpose(1, 2).to(dt))
        return 0
