"""Tidelorn: a decoder-only design with post-sum normalisation, two kinds of sink attention (global with a learned
sink and a position-dependent query gain; sliding-window with a zero sink), value mixing across layers, a clamped
gated feed-forward and a token + hashed-bigram + sinusoid embedding.

The model plugs into the same runtime as `model.Transformer`: `setup_caches` builds one `cache.KVCache*` per layer
through `get_cache_constructor` ("full" for global layers, "recent_global" without global tokens = a ring of the
window's size for sliding layers), `forward(idx, input_pos, is_prefill)` is what `generation_utils.prefill` /
`decode_one_token` / `GraphedDecoder` call, and every step (whole prompt, a portion of it, one token) goes through
`KVCache.sequence_step` and the kernels of csrc/seq.  Matrix products are cuBLAS (torch.mm) as in the Llama prefill
path; everything between them is a fused kernel of this package.  There is no CPU path.

Precision: weights, tables, cache rows and matrix-product inputs are in the compute dtype (bf16 or fp32); matrix
products accumulate and return fp32; the residual stream, norms, q, scores, softmax weights, sinks, gains, biases and
mixing coefficients are fp32 in both modes.

The mechanisms are written with their constants as arguments (`SinkAttention`, `ClampedGLU`, `PostSumNorm`,
`HashedBigramEmbedding`) so that another design can reuse them.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional

import torch
import torch.nn as nn
from torch import Tensor

from . import _lib, seq_ops
from .cache import get_cache_constructor


def _mm(a: Tensor, w: Tensor) -> Tensor:
    """a [T, K] @ w[N, K]^T -> fp32 [T, N]: cuBLAS with fp32 accumulation and fp32 output in both compute dtypes."""
    if a.dtype == torch.float32:
        return torch.mm(a, w.t())
    return torch.mm(a, w.t(), out_dtype=torch.float32)


# --------------------------------------------------------------------------------------------- configuration

@dataclass
class TidelornArgs:
    vocab_size: int
    dim: int
    layers: List[Dict[str, Any]]
    norm_eps: float
    postln_alpha: float
    embedding_scale: float
    bigram: Optional[Dict[str, int]] = None
    block_size: int = 1 << 20          # positions are sinusoidal: no table limits the length
    n_layer: int = field(init=False)

    def __post_init__(self):
        self.n_layer = len(self.layers)
        for i, layer in enumerate(self.layers):
            if layer["type"] not in ("attention", "attention_2"):
                raise ValueError(f"layer {i}: unknown mixer type {layer['type']!r}")
            if layer.get("mlp") and layer["mlp"].get("kind") != "dense":
                raise ValueError(f"layer {i}: unknown feed-forward kind {layer['mlp'].get('kind')!r}")

    @classmethod
    def from_config(cls, cfg: Dict[str, Any]):
        emb = cfg["embedding"]
        return cls(vocab_size=int(cfg["vocab"]), dim=int(cfg["width"]), layers=list(cfg["layers"]),
                   norm_eps=float(cfg["norm"]["eps"]), postln_alpha=float(cfg["postln_alpha"]),
                   embedding_scale=float(emb.get("scale", 1.0)), bigram=emb.get("bigram") or None)


# --------------------------------------------------------------------------------------------- mechanisms

class PostSumNorm(nn.Module):
    """x <- unit_rms(alpha * x + y) * (1 + weight): the gain is stored as an offset from one; fp32, in place."""

    def __init__(self, dim: int, eps: float, alpha: float = 1.0):
        super().__init__()
        self.eps, self.alpha = eps, alpha
        self.weight = nn.Parameter(torch.zeros(dim, dtype=torch.float32), requires_grad=False)

    def forward(self, x: Tensor, y: Optional[Tensor], x_act: Optional[Tensor], alpha: Optional[float] = None) -> Tensor:
        seq_ops.seq_residual_norm(x, y, self.weight, self.alpha if alpha is None else alpha, self.eps, x_act)
        return x


class HashedBigramEmbedding(nn.Module):
    """token row * scale + hashed (previous, current) row + sinusoid of the position.  The previous token of the
    running sequence is device state (`prev_token`), cleared by `reset`."""

    def __init__(self, vocab: int, dim: int, scale: float, bigram: Optional[Dict[str, int]], dtype):
        super().__init__()
        self.dim, self.scale = dim, scale
        self.weight = nn.Parameter(torch.zeros(vocab, dim, dtype=dtype), requires_grad=False)
        self.buckets = int(bigram["buckets"]) if bigram else 0
        self.mul_prev = int(bigram["mul_prev"]) if bigram else 0
        self.mul_cur = int(bigram["mul_cur"]) if bigram else 0
        self.bigram = nn.Parameter(torch.zeros(self.buckets + 1, dim, dtype=dtype), requires_grad=False) if bigram else None
        i = torch.arange(0, dim, 2, dtype=torch.float32)
        self.register_buffer("inv_freq", torch.pow(torch.tensor(10000.0, dtype=torch.float32), -i / dim), persistent=False)
        self.register_buffer("prev_token", torch.full((1,), -1, dtype=torch.int32), persistent=False)

    def reset(self):
        self.prev_token.fill_(-1)

    def forward(self, tokens: Tensor, input_pos: Tensor, x: Tensor, x_act: Optional[Tensor]) -> Tensor:
        seq_ops.seq_embed(tokens, input_pos, self.prev_token, self.weight, self.bigram, self.inv_freq, x, x_act,
                          self.scale, self.buckets, self.mul_prev, self.mul_cur)
        return x


class SinkAttention(nn.Module):
    """Grouped-query attention with fp32 scores and a sink term in the softmax denominator, over a position-addressed
    cache.  Options: projection biases, unit-RMS q/k, a query gain 1 + coef * ln(floor((p + 1) / every) + 1), a
    sliding window, a learned or a zero sink, mixing of the values with those of an earlier layer."""

    def __init__(self, dim: int, heads: int, kv_heads: int, head_dim: int, v_head_dim: int, scale: float, eps: float,
                 dtype, bias: bool = False, sink: Optional[str] = None, window: int = 0, gain_coef: float = 0.0,
                 gain_every: int = 0, v_mix: bool = False, unit_norm: bool = True):
        super().__init__()
        assert heads % kv_heads == 0 and sink in (None, "learned", "zero")
        self.dim, self.heads, self.kv_heads, self.head_dim, self.v_head_dim = dim, heads, kv_heads, head_dim, v_head_dim
        self.scale, self.eps, self.window, self.v_mix, self.unit_norm = scale, eps, int(window), v_mix, unit_norm
        self.gain_coef, self.gain_every = float(gain_coef), int(gain_every)
        self.sink_mode = {None: _lib.SINK_NONE, "learned": _lib.SINK_LEARNED, "zero": _lib.SINK_ZERO}[sink]
        n_qkv = (heads + kv_heads) * head_dim + kv_heads * v_head_dim
        self.wqkv = nn.Parameter(torch.zeros(n_qkv, dim, dtype=dtype), requires_grad=False)
        self.wo = nn.Parameter(torch.zeros(dim, heads * v_head_dim, dtype=dtype), requires_grad=False)
        self.bqkv = nn.Parameter(torch.zeros(n_qkv, dtype=torch.float32), requires_grad=False) if bias else None
        self.sink = nn.Parameter(torch.zeros(heads, dtype=torch.float32), requires_grad=False) if sink == "learned" else None
        self.vmix = nn.Parameter(torch.zeros(1, dtype=torch.float32), requires_grad=False) if v_mix else None
        self.kv_cache = None

    def forward(self, x_act: Tensor, input_pos: Tensor, v_first: Optional[Tensor]):
        """x_act [T, dim] compute dtype -> (fp32 [T, dim] mixer output, this layer's values [T, G * Dv])."""
        T = x_act.shape[0]
        H, G, Dk, Dv = self.heads, self.kv_heads, self.head_dim, self.v_head_dim
        dt, dev = self.wqkv.dtype, x_act.device
        qkv = _mm(x_act, self.wqkv)
        q = torch.empty(T, H, Dk, dtype=torch.float32, device=dev)
        k = torch.empty(T, G, Dk, dtype=dt, device=dev)
        v = torch.empty(T, G, Dv, dtype=dt, device=dev)
        mix_from = v_first if self.v_mix else None
        seq_ops.seq_qkv_prepare(qkv, self.bqkv, input_pos, self.vmix if mix_from is not None else None, mix_from, q, k, v,
                                H, G, Dk, Dv, self.eps, self.unit_norm, self.gain_coef, self.gain_every)
        y = torch.empty(T, H, Dv, dtype=dt, device=dev)
        self.kv_cache.sequence_step(q, k, v, input_pos, y, window=self.window, sink=self.sink, sink_mode=self.sink_mode,
                                    scale=self.scale)
        return _mm(y.view(T, H * Dv), self.wo), v


class ClampedGLU(nn.Module):
    """down(g * sigmoid(slope * g) * (u + 1)) with g = min(gate x, limit), u = clamp(up x, -limit, limit)."""

    def __init__(self, dim: int, ff: int, limit: float, dtype, slope: float = 1.702):
        super().__init__()
        self.ff, self.limit, self.slope = ff, float(limit), float(slope)
        self.w13 = nn.Parameter(torch.zeros(2 * ff, dim, dtype=dtype), requires_grad=False)   # rows: gate | up
        self.w2 = nn.Parameter(torch.zeros(dim, ff, dtype=dtype), requires_grad=False)

    def forward(self, x_act: Tensor) -> Tensor:
        gu = _mm(x_act, self.w13)
        act = torch.empty(x_act.shape[0], self.ff, dtype=self.w2.dtype, device=x_act.device)
        seq_ops.seq_clamped_glu(gu, act, self.limit, self.slope)
        return _mm(act, self.w2)


class TidelornBlock(nn.Module):
    def __init__(self, cfg: TidelornArgs, layer: Dict[str, Any], dtype):
        super().__init__()
        m = layer["mixer"]
        common = dict(dim=cfg.dim, heads=int(m["heads"]), kv_heads=int(m["kv_heads"]), head_dim=int(m["dim"]),
                      v_head_dim=int(m["vdim"]), scale=float(m["scale"]), eps=cfg.norm_eps, dtype=dtype,
                      v_mix=bool(m.get("v_mix", False)))
        if layer["type"] == "attention":
            qt = m.get("q_temp") or {}
            self.attention = SinkAttention(**common, bias=True, sink="learned", gain_coef=float(qt.get("coef", 0.0)),
                                           gain_every=int(qt.get("every", 0)))
        else:
            self.attention = SinkAttention(**common, bias=False, sink="zero", window=int(m["mask"]["size"]))
        self.norm1 = PostSumNorm(cfg.dim, cfg.norm_eps, cfg.postln_alpha)
        mlp = layer.get("mlp")
        self.feed_forward = ClampedGLU(cfg.dim, int(mlp["ff"]), float(mlp["limit"]), dtype) if mlp else None
        self.norm2 = PostSumNorm(cfg.dim, cfg.norm_eps, cfg.postln_alpha) if mlp else None


# --------------------------------------------------------------------------------------------- the model

class TidelornTransformer(nn.Module):
    """Same runtime surface as `model.Transformer`: setup_caches / reset_caches / forward / min_cache_length /
    get_cache_stats / prompt_cache_overflow, `config.block_size`, `config.n_layer`, `layers[i].attention.kv_cache`."""

    supports_prompt_portions = True   # forward(is_prefill=True) continues from whatever the caches hold

    def __init__(self, config: TidelornArgs, dtype=torch.bfloat16):
        super().__init__()
        assert dtype in (torch.bfloat16, torch.float32)
        self.config, self.dtype = config, dtype
        self.tok_embeddings = HashedBigramEmbedding(config.vocab_size, config.dim, config.embedding_scale, config.bigram, dtype)
        self.layers = nn.ModuleList(TidelornBlock(config, layer, dtype) for layer in config.layers)
        self.norm = PostSumNorm(config.dim, config.norm_eps, 1.0)
        self.output = nn.Parameter(torch.zeros(config.vocab_size, config.dim, dtype=dtype), requires_grad=False)
        self.max_batch_size = 1
        mixing = [b.attention for b in self.layers if b.attention.v_mix]
        widths = {a.kv_heads * a.v_head_dim for a in mixing}
        if len(widths) > 1:
            raise ValueError("layers that mix values must agree on kv_heads * vdim")
        self._first_mixing = mixing[0] if mixing else None
        # one-token steps through the fused product kernels (norm folded into the products); False = the same
        # kernels as a prompt portion of one token (library products + norm launches), used by the A/B tests
        self.fused_decode = True

    # ---- caches ---------------------------------------------------------------------------------
    def layer_cache_plan(self, cache_kwargs: Dict[str, Any], max_seq_length: int) -> Dict[str, Any]:
        """Per-layer cache kinds follow from the layer types: a global layer keeps everything ("full", one slot per
        position up to max_seq_length), a sliding layer keeps its window ("recent_global" with no global tokens)."""
        ck = dict(cache_kwargs or {})
        ck["max_seq_length"] = max_seq_length
        ck["cache_strategy"] = ["recent_global" if b.attention.window else "full" for b in self.layers]
        ck["max_cache_length"] = [b.attention.window or max_seq_length for b in self.layers]
        ck["global_tokens"] = 0
        ck["cache_bits"] = None
        ck["prompt_compression_strategy"] = ["none"] * len(self.layers)   # nothing is ever dropped from a prompt
        return ck

    def setup_caches(self, **kwargs):
        strategies, lengths = kwargs["cache_strategy"], kwargs["max_cache_length"]
        for i, block in enumerate(self.layers):
            att = block.attention
            ctor, relevant = get_cache_constructor(cache_strategy=strategies[i])
            layer_kwargs = {k: (kwargs[k][i] if k == "max_cache_length" else kwargs.get(k)) for k in relevant
                            if k in kwargs}
            layer_kwargs["max_cache_length"] = int(lengths[i])
            att.kv_cache = ctor(self.max_batch_size, att.kv_heads, att.head_dim, self.dtype, v_head_dim=att.v_head_dim,
                                **layer_kwargs)
        self.max_seq_length = int(kwargs.get("max_seq_length") or max(lengths))

    def reset_caches(self):
        """Gives back what the finished sequence held: every slot empty, no previous token."""
        for layer in self.layers:
            layer.attention.kv_cache.reset()
        self.tok_embeddings.reset()

    def prompt_cache_overflow(self, prompt_length: int):
        return [False if b.attention.window else prompt_length > b.attention.kv_cache.max_cache_length for b in self.layers]

    def min_cache_length(self):
        full = [b.attention.kv_cache.max_cache_length for b in self.layers if not b.attention.window]
        return min(full) if full else self.max_seq_length

    def get_cache_stats(self, prompt_len, gen_len):
        stats, mem = {}, 0.0
        for i, layer in enumerate(self.layers):
            c = layer.attention.kv_cache
            stats[f"cache_slots_{i}"] = float(c.max_cache_length)
            mem += c.memory_usage()
        stats["cache_memory_gb"] = mem
        return stats

    # ---- one step: a whole prompt, a portion of it, or one token ----------------------------------
    @torch.no_grad()
    def forward(self, idx: Tensor, input_pos: Tensor, is_prefill: bool = True, mask: Optional[Tensor] = None,
                attn_top_k: Optional[float] = 1.0, logits_at: Optional[Tensor] = None,
                collect: Optional[list] = None) -> Tensor:
        """idx [1, T] token ids, input_pos [T] (or [1]) positions with input_pos[0] the first token's; returns fp32
        logits [1, n, vocab] for the rows `logits_at` (positions inside this step; default: the last).  The step
        continues from what earlier steps left in the caches, so portions of any size give the same logits.  `collect`, if
        a list, receives a copy of the residual stream after every layer (diagnostics and tests)."""
        assert attn_top_k in (None, 1, 1.0), "top-k attention is not part of this design"
        if self.layers[0].attention.kv_cache is None:
            raise RuntimeError("Caches must be initialized first")
        tokens = idx.reshape(-1)
        if not tokens.is_cuda:
            raise _lib.CcError("this model runs on CUDA tensors only (no CPU fallback)")
        tokens = tokens if tokens.dtype == torch.int32 else tokens.to(torch.int32)
        ip = input_pos.reshape(-1)[:1]
        ip = ip if ip.dtype == torch.int32 else ip.to(torch.int32)
        T, E, dev = tokens.numel(), self.config.dim, tokens.device
        if T == 1 and not is_prefill and self.fused_decode and collect is None and self._fused_decode_fits():
            return self._decode_fused(tokens, ip)
        x = torch.empty(T, E, dtype=torch.float32, device=dev)
        x_act = x if self.dtype == torch.float32 else torch.empty(T, E, dtype=self.dtype, device=dev)
        side = None if x_act is x else x_act
        self.tok_embeddings(tokens, ip, x, side)
        v_first = None
        for block in self.layers:
            att = block.attention
            out, v = att(x_act, ip, v_first)
            if att is self._first_mixing:
                v_first = v
            block.norm1(x, out, side)
            if block.feed_forward is not None:
                block.norm2(x, block.feed_forward(x_act), side)
            elif block.norm2 is not None:   # a second norm without a feed-forward: x <- norm2(alpha * x)
                block.norm2(x, None, side)
            if collect is not None:
                collect.append(x.clone())
        if logits_at is None:
            xs = x[T - 1:].clone()
        else:
            xs = x.index_select(0, logits_at.to(device=dev, dtype=torch.long))
        xs_act = xs if self.dtype == torch.float32 else torch.empty_like(xs, dtype=self.dtype)
        self.norm(xs, None, None if xs_act is xs else xs_act)
        return _mm(xs_act, self.output).view(1, xs.shape[0], -1)

    def _fused_decode_fits(self) -> bool:
        """The one-token product kernel stages its input vector in shared memory (up to 51200 elements) and knows the
        two sublayer forms of a block; anything else takes the general step."""
        widest = max([self.config.dim] + [b.feed_forward.ff for b in self.layers if b.feed_forward is not None]
                     + [b.attention.heads * b.attention.v_head_dim for b in self.layers])
        return widest <= 51200 and all(b.norm2 is None or b.feed_forward is not None for b in self.layers)

    def _decode_fused(self, tokens: Tensor, ip: Tensor) -> Tensor:
        """One token with the stream kept as the pre-norm sum `s` of the last sublayer: every product reads
        `norm(s)` through its prologue and the row-parallel ones write `alpha * norm(s) + W y` through their epilogue
        (cc_seq_gemv), so no norm launch separates two products.  Per layer: qkv product, q/k/v preparation, attention +
        append, o product, gate/up product with the clamped unit, down product."""
        E, dev, dt = self.config.dim, tokens.device, self.dtype
        f32 = dict(dtype=torch.float32, device=dev)
        x0 = torch.empty(1, E, **f32)
        x0_act = x0 if dt == torch.float32 else torch.empty(1, E, dtype=dt, device=dev)
        self.tok_embeddings(tokens, ip, x0, None if x0_act is x0 else x0_act)
        cur, cur_w, cur_in = x0, None, x0_act     # the stream (a sum, or the embedding), its norm gain, what products read
        v_first = None
        gemv = seq_ops.seq_gemv
        for block in self.layers:
            att = block.attention
            H, G, Dk, Dv = att.heads, att.kv_heads, att.head_dim, att.v_head_dim
            qkv = torch.empty(1, att.wqkv.shape[0], **f32)
            gemv(cur_in, cur_w, att.wqkv, None, None, None, qkv, _lib.GEMV_PLAIN, 1.0, att.eps, 0.0, 0.0)
            q = torch.empty(1, H, Dk, **f32)
            k = torch.empty(1, G, Dk, dtype=dt, device=dev)
            v = torch.empty(1, G, Dv, dtype=dt, device=dev)
            mix_from = v_first if att.v_mix else None
            seq_ops.seq_qkv_prepare(qkv, att.bqkv, ip, att.vmix if mix_from is not None else None, mix_from, q, k, v,
                                    H, G, Dk, Dv, att.eps, att.unit_norm, att.gain_coef, att.gain_every)
            if att is self._first_mixing:
                v_first = v
            y = torch.empty(1, H, Dv, dtype=dt, device=dev)
            att.kv_cache.sequence_step(q, k, v, ip, y, window=att.window, sink=att.sink, sink_mode=att.sink_mode, scale=att.scale)
            s1 = torch.empty(1, E, **f32)
            gemv(y, None, att.wo, None, cur, cur_w, s1, _lib.GEMV_RESIDUAL, block.norm1.alpha, block.norm1.eps, 0.0, 0.0)
            cur, cur_w, cur_in = s1, block.norm1.weight, s1
            ff = block.feed_forward
            if ff is not None:
                act = torch.empty(1, ff.ff, dtype=dt, device=dev)
                gemv(s1, block.norm1.weight, ff.w13, None, None, None, act, _lib.GEMV_GLU, 1.0, block.norm1.eps, ff.limit, ff.slope)
                s2 = torch.empty(1, E, **f32)
                gemv(act, None, ff.w2, None, s1, block.norm1.weight, s2, _lib.GEMV_RESIDUAL, block.norm2.alpha, block.norm2.eps, 0.0, 0.0)
                cur, cur_w, cur_in = s2, block.norm2.weight, s2
        xs = cur.clone()
        if cur_w is not None:
            seq_ops.seq_residual_norm(xs, None, cur_w, 1.0, self.norm.eps, None)
        logits = torch.empty(1, self.config.vocab_size, **f32)
        gemv(xs, self.norm.weight, self.output, None, None, None, logits, _lib.GEMV_PLAIN, 1.0, self.norm.eps, 0.0, 0.0)
        return logits.view(1, 1, -1)

    def kernels_per_token(self) -> int:
        """Launches of this package's kernels in one decode step: embedding, per layer [qkv product, preparation,
        attention + append, o product, (gate/up product, down product)], last norm, output product."""
        if not self.fused_decode:
            return 2 + sum(3 + (2 if b.feed_forward is not None else 0) for b in self.layers)
        return 3 + sum(4 + (2 if b.feed_forward is not None else 0) for b in self.layers)

    # ---- weights --------------------------------------------------------------------------------
    def load_tensors(self, tensors: Dict[str, Tensor]):
        """Fills the parameters from the checkpoint's own tensor names ('embed', 'bigram', 'l<i>.norm1', 'l<i>.mix.q'
        (+ '.b'), '.k', '.v', '.o', '.sink', '.vmix', 'l<i>.mlp.gate' / '.up' / '.down', 'final.norm', 'head'),
        fusing q|k|v and gate|up rows."""
        used = set()

        def get(name, shape=None):
            if name not in tensors:
                raise KeyError(f"checkpoint has no tensor {name!r}")
            used.add(name)
            t = tensors[name]
            if shape is not None and tuple(t.shape) != tuple(shape):
                raise ValueError(f"{name}: shape {tuple(t.shape)} does not fit the configuration {tuple(shape)}")
            return t

        def put(param, value):
            param.data.copy_(value.to(param.dtype).reshape(param.shape))

        cfg = self.config
        put(self.tok_embeddings.weight, get("embed", (cfg.vocab_size, cfg.dim)))
        if self.tok_embeddings.bigram is not None:
            put(self.tok_embeddings.bigram, get("bigram", (self.tok_embeddings.buckets + 1, cfg.dim)))
        for i, block in enumerate(self.layers):
            a, p = block.attention, f"l{i}."
            nq, nk, nv = a.heads * a.head_dim, a.kv_heads * a.head_dim, a.kv_heads * a.v_head_dim
            put(a.wqkv, torch.cat([get(p + "mix.q", (nq, cfg.dim)), get(p + "mix.k", (nk, cfg.dim)), get(p + "mix.v", (nv, cfg.dim))]))
            if a.bqkv is not None:
                put(a.bqkv, torch.cat([get(p + "mix.q.b", (nq,)).float(), get(p + "mix.k.b", (nk,)).float(),
                                       get(p + "mix.v.b", (nv,)).float()]))
            put(a.wo, get(p + "mix.o", (cfg.dim, a.heads * a.v_head_dim)))
            if a.sink is not None:
                put(a.sink, get(p + "mix.sink", (a.heads,)).float())
            if a.vmix is not None:
                put(a.vmix, get(p + "mix.vmix").float())
            put(block.norm1.weight, get(p + "norm1", (cfg.dim,)).float())
            if block.feed_forward is not None:
                f = block.feed_forward
                put(f.w13, torch.cat([get(p + "mlp.gate", (f.ff, cfg.dim)), get(p + "mlp.up", (f.ff, cfg.dim))]))
                put(f.w2, get(p + "mlp.down", (cfg.dim, f.ff)))
                put(block.norm2.weight, get(p + "norm2", (cfg.dim,)).float())
            elif p + "norm2" in tensors:
                # the checkpoint carries a second norm for a layer without feed-forward: it is applied to alpha * x
                block.norm2 = PostSumNorm(cfg.dim, cfg.norm_eps, cfg.postln_alpha).to(block.norm1.weight.device)
                put(block.norm2.weight, get(p + "norm2", (cfg.dim,)).float())
        put(self.norm.weight, get("final.norm", (cfg.dim,)).float())
        put(self.output, get("head", (cfg.vocab_size, cfg.dim)))
        return sorted(set(tensors) - used)

    @classmethod
    def from_config(cls, cfg: Dict[str, Any], dtype=torch.bfloat16):
        return cls(TidelornArgs.from_config(cfg), dtype)
