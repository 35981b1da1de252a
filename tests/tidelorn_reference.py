"""Plain, slow restatement of the Tidelorn design for the tests: one function per mechanism, whole sequences at
once, dense masks, no cache, no kernels.  Everything runs on the CPU in the dtype of the tensors it is given
(the tests pass float64 or float32).  Nothing here is imported by the package.

Notation: T tokens, E model width, H query heads, G key/value heads, Dk / Dv per-head key / value sizes.
"""
from __future__ import annotations

import math

import torch


def rms_unit(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / torch.sqrt(x.pow(2).mean(-1, keepdim=True) + eps)


def zero_centred_norm(x, w, eps):
    """Unit RMS, then a gain stored as an offset from one."""
    return rms_unit(x, eps) * (1.0 + w)


def sinusoid(positions, width, dtype):
    """[T, E]: even entries sin(p * w_i), odd entries cos(p * w_i), w_i = 10000^(-2i/E)."""
    i = torch.arange(0, width, 2, dtype=dtype)
    w = torch.pow(torch.tensor(10000.0, dtype=dtype), -i / width)
    ang = positions.to(dtype)[:, None] * w[None, :]
    out = torch.zeros(len(positions), width, dtype=dtype)
    out[:, 0::2] = torch.sin(ang)[:, : out[:, 0::2].shape[1]]
    out[:, 1::2] = torch.cos(ang)[:, : out[:, 1::2].shape[1]]
    return out


def bigram_rows(tokens, buckets, mul_prev, mul_cur):
    """Hashed (previous, current) row per token; the first token of a sequence takes the extra last row."""
    rows = [buckets]
    for a, b in zip(tokens[:-1], tokens[1:]):
        rows.append((int(a) * mul_prev + int(b) * mul_cur) % buckets)
    return torch.tensor(rows[: len(tokens)], dtype=torch.long)


def embed(tokens, W, cfg):
    e = cfg["embedding"]
    dtype = W["embed"].dtype
    tok = torch.as_tensor(tokens, dtype=torch.long)
    x = W["embed"][tok] * e["scale"]
    if "bigram" in e and e["bigram"]:
        b = e["bigram"]
        x = x + W["bigram"][bigram_rows(list(tokens), b["buckets"], b["mul_prev"], b["mul_cur"])]
    return x + sinusoid(torch.arange(len(tok)), x.shape[-1], dtype)


def query_temperature(T, coef, every, dtype):
    p = torch.arange(T)
    return 1.0 + coef * torch.log((torch.div(p + 1, every, rounding_mode="floor") + 1).to(dtype))


def sink_softmax(scores, allowed, sink):
    """Row softmax over the allowed keys with one extra, value-less logit per row in the denominator.
    scores [H, T, T], allowed [T, T] bool, sink [H] (or a scalar)."""
    s = scores.masked_fill(~allowed, float("-inf"))
    sink = torch.as_tensor(sink, dtype=scores.dtype).reshape(-1, 1, 1).expand(s.shape[0], s.shape[1], 1)
    m = torch.maximum(s.max(-1, keepdim=True).values, sink)
    e = torch.exp(s - m)
    return e / (e.sum(-1, keepdim=True) + torch.exp(sink - m))


def attention_mixer(h, W, pfx, m, eps, kind, v_first):
    """One attention mixer over a whole sequence.  kind 'attention': biases, learned sink, query temperature,
    causal.  kind 'attention_2': no biases, sink logit 0, sliding window.  Returns (out, v) with v the values after
    mixing (what later layers would see as this layer's cached values)."""
    T = h.shape[0]
    H, G, Dk, Dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q, k, v = h @ W[pfx + "q"].T, h @ W[pfx + "k"].T, h @ W[pfx + "v"].T
    if kind == "attention":
        q, k, v = q + W[pfx + "q.b"], k + W[pfx + "k.b"], v + W[pfx + "v.b"]
    if m.get("v_mix") and v_first is not None:
        lam = W[pfx + "vmix"]
        v = (1.0 - lam) * v + lam * v_first
    q = rms_unit(q.view(T, H, Dk), eps)
    k = rms_unit(k.view(T, G, Dk), eps)
    if kind == "attention" and m.get("q_temp"):
        q = q * query_temperature(T, m["q_temp"]["coef"], m["q_temp"]["every"], h.dtype)[:, None, None]
    kk = k.repeat_interleave(H // G, dim=1)
    vv = v.view(T, G, Dv).repeat_interleave(H // G, dim=1)
    scores = torch.einsum("ihd,jhd->hij", q, kk) * m["scale"]
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    allowed = j <= i
    if kind == "attention_2":
        allowed = allowed & (i - j < m["mask"]["size"])
        sink = torch.zeros(H, dtype=h.dtype)
    else:
        sink = W[pfx + "sink"]
    p = sink_softmax(scores, allowed, sink)
    y = torch.einsum("hij,jhd->ihd", p, vv).reshape(T, H * Dv)
    return y @ W[pfx + "o"].T, v


def clamped_glu(h, W, pfx, mlp):
    lim = mlp["limit"]
    g = torch.clamp(h @ W[pfx + "gate"].T, max=lim)
    u = torch.clamp(h @ W[pfx + "up"].T, -lim, lim)
    return (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ W[pfx + "down"].T


def forward(tokens, W, cfg, collect=None):
    """Logits [T, vocab] of one whole sequence.  `collect`, if a list, receives the stream after every layer."""
    eps, alpha = cfg["norm"]["eps"], cfg["postln_alpha"]
    x = embed(tokens, W, cfg)
    v_first = None
    for li, layer in enumerate(cfg["layers"]):
        pfx = f"l{li}."
        out, v = attention_mixer(x, W, pfx + "mix.", layer["mixer"], eps, layer["type"], v_first)
        if layer["mixer"].get("v_mix") and v_first is None:
            v_first = v
        x = zero_centred_norm(alpha * x + out, W[pfx + "norm1"], eps)
        if layer.get("mlp"):
            x = zero_centred_norm(alpha * x + clamped_glu(x, W, pfx + "mlp.", layer["mlp"]), W[pfx + "norm2"], eps)
        elif pfx + "norm2" in W:   # a checkpoint that carries a second norm for a layer without feed-forward
            x = zero_centred_norm(alpha * x, W[pfx + "norm2"], eps)
        if collect is not None:
            collect.append(x.clone())
    return zero_centred_norm(x, W["final.norm"], eps) @ W["head"].T
