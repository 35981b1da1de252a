"""PyTorch custom ops over the sequence-kernel C ABI (include/cc_b200_seq.h, libcc_b200_seq.so).

Registered in the same `torch.ops.cold_compress_b200` namespace as the compressed-KV ops (ops.py), with schemas that
declare the in-place writes.  CUDA tensors only: the CPU registrations raise.  Element types are taken from the
tensors: fp32 or bf16 for activations, tables and cache rows; the residual stream, q, sinks, biases, norm gains and
mixing coefficients are always fp32.
"""
from __future__ import annotations

import ctypes as C

import torch

from . import _lib

_library = torch.library.Library("cold_compress_b200", "FRAGMENT")

ATTN_CHUNK, ATTN_DECODE_APPEND, ATTN_APPEND_ONLY, ATTN_DECODE = 0, 1, 2, 3

_library.define("seq_embed(Tensor tokens, Tensor input_pos, Tensor(a!) prev_token, Tensor embed, Tensor? bigram, "
                "Tensor inv_freq, Tensor(b!) x, Tensor(c!)? x_act, float scale, int buckets, int mul_prev, int mul_cur) -> ()")
_library.define("seq_qkv_prepare(Tensor qkv, Tensor? bias, Tensor input_pos, Tensor? mix_lambda, Tensor? v_first, "
                "Tensor(a!) q, Tensor(b!) k, Tensor(c!) v, int H, int G, int Dk, int Dv, float eps, bool unit_norm, "
                "float gain_coef, int gain_every) -> ()")
_library.define("seq_attention(Tensor q, Tensor k_new, Tensor v_new, Tensor(a!) k_cache, Tensor(b!) v_cache, Tensor(c!) pos, "
                "Tensor(d!) mask, Tensor(e!) cache_cts, Tensor input_pos, Tensor(f!) y, Tensor? sink, int window, "
                "int sink_mode, float scale, int mode, Tensor(g!)? workspace) -> ()")
_library.define("seq_residual_norm(Tensor(a!) x, Tensor? y, Tensor w, float alpha, float eps, Tensor(b!)? x_act) -> ()")
_library.define("seq_clamped_glu(Tensor gu, Tensor(a!) out, float limit, float slope) -> ()")
_library.define("seq_gemv(Tensor x, Tensor? in_norm_w, Tensor w, Tensor? bias, Tensor? res, Tensor? res_norm_w, Tensor(a!) out, "
                "int mode, float alpha, float eps, float limit, float slope) -> ()")


def _dt(t: torch.Tensor) -> int:
    if t.dtype == torch.float32:
        return _lib.DT_F32
    if t.dtype == torch.bfloat16:
        return _lib.DT_BF16
    raise _lib.CcError(f"sequence kernels take fp32 or bf16 tensors, not {t.dtype}")


def _p(t):
    return None if t is None else t.data_ptr()


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _need(*pairs):
    for name, t, dtype in pairs:
        if t is None:
            continue
        if not t.is_cuda:
            raise _lib.CcError("cold_compress_b200 sequence ops run on CUDA tensors only (no CPU fallback)")
        if not t.is_contiguous():
            raise _lib.CcError(f"{name}: expected a contiguous tensor")
        if dtype is not None and t.dtype != dtype:
            raise _lib.CcError(f"{name}: expected {dtype}, got {t.dtype}")


def _seq_embed(tokens, input_pos, prev_token, embed, bigram, inv_freq, x, x_act, scale, buckets, mul_prev, mul_cur):
    _need(("tokens", tokens, torch.int32), ("input_pos", input_pos, torch.int32), ("prev_token", prev_token, torch.int32),
          ("embed", embed, None), ("bigram", bigram, embed.dtype), ("inv_freq", inv_freq, torch.float32),
          ("x", x, torch.float32), ("x_act", x_act, None))
    T, E = tokens.numel(), embed.shape[1]
    assert x.shape[-1] == E and x.numel() == T * E and inv_freq.numel() >= (E + 1) // 2
    _lib.check_seq(_lib.load_seq().cc_seq_embed(
        _p(tokens), _p(input_pos), _p(prev_token), _p(embed), _p(bigram), _p(inv_freq), _p(x), _p(x_act), T, E,
        float(scale), int(buckets), int(mul_prev), int(mul_cur), _dt(embed), _dt(x_act) if x_act is not None else _lib.DT_F32,
        _stream()), "cc_seq_embed")


def _seq_qkv_prepare(qkv, bias, input_pos, mix_lambda, v_first, q, k, v, H, G, Dk, Dv, eps, unit_norm, gain_coef, gain_every):
    _need(("qkv", qkv, None), ("bias", bias, torch.float32), ("input_pos", input_pos, torch.int32),
          ("mix_lambda", mix_lambda, torch.float32), ("v_first", v_first, k.dtype), ("q", q, torch.float32), ("k", k, None),
          ("v", v, k.dtype))
    T = qkv.shape[0]
    assert qkv.shape[1] == (H + G) * Dk + G * Dv and q.numel() == T * H * Dk and k.numel() == T * G * Dk and v.numel() == T * G * Dv
    _lib.check_seq(_lib.load_seq().cc_seq_qkv_prepare(
        _p(qkv), _dt(qkv), _p(bias), _p(input_pos), _p(mix_lambda), _p(v_first), _p(q), _p(k), _p(v), _dt(k), T, H, G, Dk, Dv,
        float(eps), int(bool(unit_norm)), float(gain_coef), int(gain_every), _stream()), "cc_seq_qkv_prepare")


def _seq_attention(q, k_new, v_new, k_cache, v_cache, pos, mask, cache_cts, input_pos, y, sink, window, sink_mode, scale,
                   mode, workspace):
    _need(("q", q, torch.float32), ("k_new", k_new, k_cache.dtype), ("v_new", v_new, k_cache.dtype), ("k_cache", k_cache, None),
          ("v_cache", v_cache, k_cache.dtype), ("pos", pos, torch.int32), ("mask", mask, torch.bool),
          ("cache_cts", cache_cts, torch.int32), ("input_pos", input_pos, torch.int32), ("y", y, None),
          ("sink", sink, torch.float32), ("workspace", workspace, None))
    a = _lib.CcSeqAttn()
    T, H, Dk = q.shape
    G, L = k_cache.shape[-3], k_cache.shape[-2]
    Dv = v_cache.shape[-1]
    assert k_cache.shape[-1] == Dk and k_new.shape == (T, G, Dk) and v_new.shape == (T, G, Dv) and y.shape == (T, H, Dv)
    assert pos.numel() == L and mask.numel() == G * L
    a.q, a.k_new, a.v_new, a.k_cache, a.v_cache = _p(q), _p(k_new), _p(v_new), _p(k_cache), _p(v_cache)
    a.pos, a.mask, a.cache_cts, a.input_pos, a.y, a.sink = _p(pos), _p(mask), _p(cache_cts), _p(input_pos), _p(y), _p(sink)
    a.T, a.H, a.G, a.Dk, a.Dv, a.L = T, H, G, Dk, Dv, L
    a.window, a.sink_mode, a.cache_dtype, a.y_dtype, a.scale = int(window), int(sink_mode), _dt(k_cache), _dt(y), float(scale)
    a.append = int(mode == ATTN_DECODE_APPEND)
    if workspace is not None:
        a.workspace, a.workspace_bytes = workspace.data_ptr(), workspace.numel() * workspace.element_size()
    lib = _lib.load_seq()
    if mode == ATTN_CHUNK:
        _lib.check_seq(lib.cc_seq_attention(C.byref(a), _stream()), "cc_seq_attention")
    elif mode in (ATTN_DECODE_APPEND, ATTN_DECODE):
        _lib.check_seq(lib.cc_seq_attention_decode(C.byref(a), _stream()), "cc_seq_attention_decode")
    elif mode == ATTN_APPEND_ONLY:
        _lib.check_seq(lib.cc_seq_cache_append(C.byref(a), _stream()), "cc_seq_cache_append")
    else:
        raise _lib.CcError(f"seq_attention: unknown mode {mode}")


def decode_workspace_bytes(H, G, Dv, L, window) -> int:
    return int(_lib.load_seq().cc_seq_decode_workspace(H, G, Dv, L, window))


def _seq_residual_norm(x, y, w, alpha, eps, x_act):
    _need(("x", x, torch.float32), ("y", y, None), ("w", w, torch.float32), ("x_act", x_act, None))
    E = x.shape[-1]
    T = x.numel() // E
    assert w.numel() == E and (y is None or y.numel() == x.numel()) and (x_act is None or x_act.numel() == x.numel())
    _lib.check_seq(_lib.load_seq().cc_seq_residual_norm(
        _p(x), _p(y), _dt(y) if y is not None else _lib.DT_F32, _p(w), float(alpha), float(eps), _p(x_act),
        _dt(x_act) if x_act is not None else _lib.DT_F32, T, E, _stream()), "cc_seq_residual_norm")


def _seq_clamped_glu(gu, out, limit, slope):
    _need(("gu", gu, None), ("out", out, None))
    F = out.shape[-1]
    T = out.numel() // F
    assert gu.numel() == 2 * T * F
    _lib.check_seq(_lib.load_seq().cc_seq_clamped_glu(_p(gu), _p(out), _dt(gu), _dt(out), float(limit), float(slope), T, F,
                                                      _stream()), "cc_seq_clamped_glu")


def _seq_gemv(x, in_norm_w, w, bias, res, res_norm_w, out, mode, alpha, eps, limit, slope):
    """One-token product with the post-sum norm folded into its prologue / epilogue (cc_seq_gemv)."""
    _need(("x", x, None), ("in_norm_w", in_norm_w, torch.float32), ("w", w, None), ("bias", bias, torch.float32),
          ("res", res, torch.float32), ("res_norm_w", res_norm_w, torch.float32), ("out", out, None))
    g = _lib.CcSeqGemv()
    rows, K = w.shape
    N = rows // 2 if mode == _lib.GEMV_GLU else rows
    assert x.numel() == K and out.numel() == N and (res is None or res.numel() == N) and (in_norm_w is None or in_norm_w.numel() == K)
    g.x, g.x_dtype, g.in_norm_w, g.W, g.w_dtype = _p(x), _dt(x), _p(in_norm_w), _p(w), _dt(w)
    g.bias, g.res, g.res_norm_w = _p(bias), _p(res), _p(res_norm_w)
    g.alpha, g.eps, g.limit, g.slope, g.mode = float(alpha), float(eps), float(limit), float(slope), int(mode)
    g.out, g.out_dtype, g.N, g.K = _p(out), _dt(out), N, K
    _lib.check_seq(_lib.load_seq().cc_seq_gemv(C.byref(g), _stream()), "cc_seq_gemv")


def _no_cpu(*_a, **_k):
    raise _lib.CcError("cold_compress_b200 sequence ops have no CPU implementation (sm_100a only)")


for _name, _fn in (("seq_embed", _seq_embed), ("seq_qkv_prepare", _seq_qkv_prepare), ("seq_attention", _seq_attention),
                   ("seq_residual_norm", _seq_residual_norm), ("seq_clamped_glu", _seq_clamped_glu), ("seq_gemv", _seq_gemv)):
    _library.impl(_name, _fn, "CUDA")
    _library.impl(_name, _no_cpu, "CPU")

seq_embed = torch.ops.cold_compress_b200.seq_embed
seq_qkv_prepare = torch.ops.cold_compress_b200.seq_qkv_prepare
seq_attention = torch.ops.cold_compress_b200.seq_attention
seq_residual_norm = torch.ops.cold_compress_b200.seq_residual_norm
seq_clamped_glu = torch.ops.cold_compress_b200.seq_clamped_glu
seq_gemv = torch.ops.cold_compress_b200.seq_gemv
