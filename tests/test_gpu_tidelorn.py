"""GPU tests of the Tidelorn design: every mechanism's kernel against the plain restatement in tidelorn_reference.py
(float64, CPU, whole sequences, dense masks), then the model through the runtime: prompt against token-by-token
decoding, prompt portions of many sizes, caches that are emptied and used again, window and split edges, spikes that
make one far key decide the output, other sizes, greedy generation through generate() and the graph-captured decoder."""
import math

import pytest
import torch

import tidelorn_reference as R
from tidelorn_utils import (as_double, build_model, default_layers, fp32_tolerance, global_layer, make_config,
                            random_weights, row_error, window_layer)

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _ops():
    from cold_compress_b200 import seq_ops
    return seq_ops


def _i32(*v):
    return torch.tensor(v, dtype=torch.int32, device=DEV)


# ----------------------------------------------------------------------------------------------- single mechanisms

@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_embedding_kernel_portions_and_state(dtype):
    ops = _ops()
    cfg = make_config([], width=50, vocab=97, scale=3.25, bigram=(31, 7, 11))
    g = torch.Generator().manual_seed(1)
    W = {"embed": torch.randn(97, 50, generator=g).to(torch.bfloat16), "bigram": torch.randn(32, 50, generator=g).to(torch.bfloat16)}
    tokens = torch.randint(0, 97, (23,), generator=g).tolist()
    want = R.embed(tokens, as_double(W), cfg)
    inv_freq = torch.pow(torch.tensor(10000.0), -torch.arange(0, 50, 2, dtype=torch.float32) / 50).to(DEV)
    prev = torch.full((1,), -1, dtype=torch.int32, device=DEV)
    emb, big = W["embed"].to(DEV, dtype), W["bigram"].to(DEV, dtype)
    got, at = [], 0
    for n in (1, 2, 7, 1, 12):   # the previous token crosses every portion border through `prev`
        x = torch.empty(n, 50, device=DEV)
        xa = torch.empty(n, 50, device=DEV, dtype=torch.bfloat16)
        ops.seq_embed(_i32(*tokens[at:at + n]), _i32(at), prev, emb, big, inv_freq, x, xa, 3.25, 31, 7, 11)
        assert torch.equal(xa, x.to(torch.bfloat16))
        got.append(x)
        at += n
    assert prev.item() == tokens[-1]
    err = (torch.cat(got).cpu().double() - want).abs().max().item()
    assert err < 2e-5, err
    # without the bigram table only token row and sinusoid remain
    x = torch.empty(23, 50, device=DEV)
    ops.seq_embed(_i32(*tokens), _i32(0), prev, emb, None, inv_freq, x, None, 3.25, 0, 0, 0)
    cfg2 = make_config([], width=50, vocab=97, scale=3.25, bigram=None)
    assert (x.cpu().double() - R.embed(tokens, as_double(W), cfg2)).abs().max().item() < 2e-5


def test_sinusoid_far_positions():
    ops = _ops()
    E = 36
    inv_freq = torch.pow(torch.tensor(10000.0), -torch.arange(0, E, 2, dtype=torch.float32) / E).to(DEV)
    emb = torch.zeros(4, E, device=DEV)
    x = torch.empty(3, E, device=DEV)
    ops.seq_embed(_i32(1, 2, 3), _i32(40000), torch.zeros(1, dtype=torch.int32, device=DEV), emb, None, inv_freq, x, None, 1.0, 0, 0, 0)
    p = torch.arange(40000, 40003, dtype=torch.float32)[:, None] * inv_freq.cpu()[None, :]   # fp32 angles, as the design says
    assert (x.cpu()[:, 0::2] - torch.sin(p.double())).abs().max() < 1e-5
    assert (x.cpu()[:, 1::2] - torch.cos(p.double())).abs().max() < 1e-5


@pytest.mark.parametrize("in_dtype,out_dtype", [(torch.float32, torch.float32), (torch.float32, torch.bfloat16)])
def test_qkv_prepare_kernel(in_dtype, out_dtype):
    ops = _ops()
    T, H, G, Dk, Dv, eps = 9, 6, 3, 20, 12, 1e-3
    g = torch.Generator().manual_seed(2)
    qkv = torch.randn(T, (H + G) * Dk + G * Dv, generator=g)
    bias = torch.randn(qkv.shape[1], generator=g) * 0.5
    vf = torch.randn(T, G * Dv, generator=g).to(out_dtype)
    lam, coef, every, p0 = 0.3125, 0.45, 4, 6
    q = torch.empty(T, H, Dk, device=DEV)
    k = torch.empty(T, G, Dk, device=DEV, dtype=out_dtype)
    v = torch.empty(T, G, Dv, device=DEV, dtype=out_dtype)
    ops.seq_qkv_prepare(qkv.to(DEV, in_dtype), bias.to(DEV), _i32(p0), torch.tensor([lam], device=DEV), vf.to(DEV), q, k, v,
                        H, G, Dk, Dv, eps, True, coef, every)
    z = qkv.double() + bias.double()
    zq, zk, zv = z[:, :H * Dk].view(T, H, Dk), z[:, H * Dk:(H + G) * Dk].view(T, G, Dk), z[:, (H + G) * Dk:]
    pos = torch.arange(p0, p0 + T)
    gain = 1.0 + coef * torch.log((torch.div(pos + 1, every, rounding_mode="floor") + 1).double())
    tol = 1e-5 if out_dtype == torch.float32 else 1e-2
    assert (q.cpu().double() - R.rms_unit(zq, eps) * gain[:, None, None]).abs().max() < 1e-5
    assert (k.cpu().double() - R.rms_unit(zk, eps)).abs().max() < tol
    assert (v.cpu().double().view(T, -1) - ((1 - lam) * zv + lam * vf.double())).abs().max() < tol
    # no bias, no norm, no gain, no mixing: a plain split
    ops.seq_qkv_prepare(qkv.to(DEV, in_dtype), None, _i32(p0), None, None, q, k, v, H, G, Dk, Dv, eps, False, 0.0, 0)
    assert (q.cpu().view(T, -1) - qkv[:, :H * Dk]).abs().max() < 1e-6


def test_post_sum_norm_and_clamped_glu_kernels():
    ops = _ops()
    g = torch.Generator().manual_seed(3)
    T, E, F = 5, 77, 45
    x, y, w = torch.randn(T, E, generator=g), torch.randn(T, E, generator=g), torch.randn(E, generator=g) * 0.3
    want = R.zero_centred_norm(2.25 * x.double() + y.double(), w.double(), 1e-4)
    xd = x.to(DEV).clone()
    xa = torch.empty(T, E, device=DEV, dtype=torch.bfloat16)
    ops.seq_residual_norm(xd, y.to(DEV), w.to(DEV), 2.25, 1e-4, xa)
    assert (xd.cpu().double() - want).abs().max() < 1e-5 and torch.equal(xa, xd.to(torch.bfloat16))
    xd = x.to(DEV).clone()
    ops.seq_residual_norm(xd, None, w.to(DEV), 1.0, 1e-4, None)
    assert (xd.cpu().double() - R.zero_centred_norm(x.double(), w.double(), 1e-4)).abs().max() < 1e-5
    gu = torch.randn(T, 2 * F, generator=g) * 2.0    # many values beyond the limit on both sides
    out = torch.empty(T, F, device=DEV)
    ops.seq_clamped_glu(gu.to(DEV), out, 0.75, 1.702)
    gate, up = gu[:, :F].double().clamp(max=0.75), gu[:, F:].double().clamp(-0.75, 0.75)
    assert (out.cpu().double() - gate * torch.sigmoid(1.702 * gate) * (up + 1)).abs().max() < 1e-6


def _dense_attention(q, k, v, window, sink, scale):
    """float64 attention of positions 0..T-1 with the restatement's sink softmax; q [T,H,Dk], k [T,G,Dk], v [T,G,Dv]."""
    T, H, _ = q.shape
    G = k.shape[1]
    kk, vv = k.repeat_interleave(H // G, 1), v.repeat_interleave(H // G, 1)
    s = torch.einsum("ihd,jhd->hij", q, kk) * scale
    i, j = torch.arange(T)[:, None], torch.arange(T)[None, :]
    ok = (j <= i) & ((i - j < window) if window else torch.ones_like(j <= i))
    if sink is None:
        p = torch.softmax(s.masked_fill(~ok, float("-inf")), -1)
    else:
        p = R.sink_softmax(s, ok, sink)
    return torch.einsum("hij,jhd->ihd", p, vv)


class _Cache:
    """A bare position-addressed cache (the buffers KVCache holds) for the kernel-level tests."""

    def __init__(self, G, L, Dk, Dv, dtype):
        self.k = torch.zeros(1, G, L, Dk, device=DEV, dtype=dtype)
        self.v = torch.zeros(1, G, L, Dv, device=DEV, dtype=dtype)
        self.pos = torch.full((1, 1, L), -1, dtype=torch.int32, device=DEV)
        self.mask = torch.zeros(1, G, 1, L, dtype=torch.bool, device=DEV)
        self.cts = torch.zeros(1, dtype=torch.int32, device=DEV)
        self.ws = None

    def step(self, q, k, v, p0, window, sink, sink_mode, scale, ydtype=torch.float32):
        ops = _ops()
        T, H, _ = q.shape
        y = torch.empty(T, H, v.shape[-1], device=DEV, dtype=ydtype)
        args = (q, k, v, self.k, self.v, self.pos, self.mask, self.cts, _i32(p0), y, sink, window, sink_mode, scale)
        if T == 1:
            if self.ws is None:
                n = ops.decode_workspace_bytes(H, k.shape[1], v.shape[-1], self.k.shape[2], window)
                self.ws = torch.zeros((n + 3) // 4, dtype=torch.int32, device=DEV)
            ops.seq_attention(*args, ops.ATTN_DECODE_APPEND, self.ws)
        else:
            ops.seq_attention(*args, ops.ATTN_CHUNK, None)
            ops.seq_attention(*args, ops.ATTN_APPEND_ONLY, None)
        return y


ATTN_CASES = [
    # T, H, G, Dk, Dv, window, sink, portions
    (150, 4, 2, 24, 16, 0, "learned", (150,)),
    (150, 4, 2, 24, 16, 0, "learned", (64, 1, 1, 63, 2, 19)),
    (200, 6, 2, 40, 24, 65, "zero", (200,)),
    (200, 6, 2, 40, 24, 65, "zero", (3, 64, 65, 66, 1, 1)),
    (200, 2, 2, 72, 136, 64, "zero", (130, 70)),           # wide values: the 256-column tile
    (90, 3, 1, 17, 5, 1, "zero", (40, 1, 49)),             # a window of one: only the token itself
    (300, 8, 8, 16, 48, 7, None, (2,) * 150),              # no sink, two tokens at a time through a ring of 7
    (620, 2, 1, 32, 32, 0, "learned", (300,) + (1,) * 320),    # decoding over more than two key splits
    (400, 4, 4, 8, 8, 300, "zero", (10,) + (1,) * 390),    # a window longer than one key split, wrapping the ring
]


@pytest.mark.parametrize("case", ATTN_CASES, ids=[f"T{c[0]}_H{c[1]}G{c[2]}_d{c[3]}v{c[4]}_w{c[5]}_{c[6]}_{len(c[7])}p" for c in ATTN_CASES])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_attention_kernels_against_dense(case, dtype):
    T, H, G, Dk, Dv, window, sink_kind, portions = case
    assert sum(portions) == T
    g = torch.Generator().manual_seed(T + Dk)
    q = torch.nn.functional.normalize(torch.randn(T, H, Dk, generator=g), dim=-1) * math.sqrt(Dk)
    k = (torch.nn.functional.normalize(torch.randn(T, G, Dk, generator=g), dim=-1) * math.sqrt(Dk)).to(dtype)
    v = torch.randn(T, G, Dv, generator=g).to(dtype)
    sink = torch.randn(H, generator=g) if sink_kind == "learned" else None
    scale = 2.0 / math.sqrt(Dk)
    mode = {"learned": 1, "zero": 2, None: 0}[sink_kind]
    sink_ref = {"learned": sink.double() if sink is not None else None, "zero": torch.zeros(H, dtype=torch.float64), None: None}[sink_kind]
    want = _dense_attention(q.double(), k.double(), v.double(), window, sink_ref, scale)
    L = window if window else T + 3
    cache = _Cache(G, L, Dk, Dv, dtype)
    got, at = [], 0
    for n in portions:
        got.append(cache.step(q[at:at + n].to(DEV), k[at:at + n].to(DEV), v[at:at + n].to(DEV), at, window,
                              sink.to(DEV) if sink is not None else None, mode, scale))
        at += n
    got = torch.cat(got).cpu().double()
    assert (got - want).abs().max() < 2e-5, (got - want).abs().max()
    filled = min(T, L)
    assert cache.cts.item() == filled and int(cache.mask.sum()) == filled * G
    assert sorted(cache.pos.view(-1).tolist())[-filled:] == list(range(T - filled, T))


@pytest.mark.parametrize("decode", [False, True])
@pytest.mark.parametrize("window,dist,seen", [(0, 700, True), (50, 49, True), (50, 50, False), (257, 256, True), (257, 257, False)])
def test_one_far_key_decides(window, dist, seen, decode):
    """All keys but one are orthogonal to the query; the one at distance `dist` is aligned with it and carries a value
    nobody else has.  The output is that value iff the key is inside the window (or there is no window)."""
    T, Dk, Dv = dist + 40, 16, 8
    last = T - 1
    star = last - dist
    q = torch.zeros(T, 1, Dk)
    k = torch.zeros(T, 1, Dk)
    v = torch.zeros(T, 1, Dv)
    k[:, 0, 1] = 4.0
    q[:, 0, 0] = 4.0
    k[star, 0, 0] = 4.0
    v[star, 0, :] = 1.0
    cache = _Cache(1, window if window else T, Dk, Dv, torch.float32)
    portions = [T - 1, 1] if decode else [star + 3, T - star - 3]
    at, y = 0, None
    for n in portions:
        y = cache.step(q[at:at + n].to(DEV), k[at:at + n].to(DEV), v[at:at + n].to(DEV), at, window, None, 2, 2.0)
        at += n
    out = y[-1, 0].cpu()
    if seen:
        assert out.min() > 0.99, out
    else:
        assert out.abs().max() < 1e-6, out


def test_stale_slots_are_not_keys():
    """After a reset that only clears the slot positions, old rows left in the buffers must not be attended to."""
    g = torch.Generator().manual_seed(5)
    T, Dk, Dv = 40, 16, 8
    cache = _Cache(1, 64, Dk, Dv, torch.float32)
    junk = torch.randn(60, 1, Dk, generator=g) * 3
    cache.step(junk.to(DEV), junk.to(DEV), torch.randn(60, 1, Dv, generator=g).to(DEV) * 50, 0, 0, None, 2, 1.0)
    cache.pos.fill_(-1)
    cache.mask.zero_()
    cache.cts.zero_()
    q, k, v = torch.randn(T, 1, Dk, generator=g), torch.randn(T, 1, Dk, generator=g), torch.randn(T, 1, Dv, generator=g)
    y1 = cache.step(q[:25].to(DEV), k[:25].to(DEV), v[:25].to(DEV), 0, 0, None, 2, 0.5)
    y2 = cache.step(q[25:].to(DEV), k[25:].to(DEV), v[25:].to(DEV), 25, 0, None, 2, 0.5)
    want = _dense_attention(q.double(), k.double(), v.double(), 0, torch.zeros(1, dtype=torch.float64), 0.5)
    assert (torch.cat([y1, y2]).cpu().double() - want).abs().max() < 1e-5


# ----------------------------------------------------------------------------------------------- the model

def _reference_logits(cfg, W, tokens, collect=None):
    return R.forward(tokens, as_double(W), cfg, collect)


def _run_portions(model, tokens, portions, want_all=True):
    from cold_compress_b200.generation_utils import model_step
    out, at = [], 0
    for n in portions:
        x = torch.tensor(tokens[at:at + n], dtype=torch.int32, device=DEV).view(1, -1)
        ip = torch.arange(at, at + n, dtype=torch.int32, device=DEV)
        out.append(model_step(model, x, ip, is_prefill=not (n == 1 and at > 0), logits_at=torch.arange(n, device=DEV))[0])
        at += n
    return torch.cat(out)


BF16_TOL = 6e-2   # bf16 matrix-product inputs and cache rows through a handful of layers


def _tol(dtype, cfg, W, tokens, want):
    return fp32_tolerance(cfg, W, tokens, want) if dtype == torch.float32 else BF16_TOL


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_layers_one_by_one_and_logits(dtype):
    cfg = make_config(default_layers())
    W = random_weights(cfg, seed=7)
    tokens = torch.randint(0, cfg["vocab"], (61,), generator=torch.Generator().manual_seed(8)).tolist()
    ref_layers = []
    want = _reference_logits(cfg, W, tokens, ref_layers)
    model = build_model(cfg, W, dtype, 64)
    got_layers = []
    x = torch.tensor(tokens, dtype=torch.int32, device=DEV).view(1, -1)
    got = model(x, torch.arange(61, dtype=torch.int32, device=DEV), True, logits_at=torch.arange(61), collect=got_layers)[0]
    assert len(got_layers) == len(ref_layers)
    tol = _tol(dtype, cfg, W, tokens, want)
    for i, (a, b) in enumerate(zip(got_layers, ref_layers)):
        assert row_error(a, b).max() < tol, f"layer {i}: {row_error(a, b).max()}"
    assert row_error(got, want).max() < tol


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("portions", [(1,) * 70, (70,), (2,) * 35, (3, 11, 1, 1, 37, 2, 2, 12, 1), (36, 1, 33), (69, 1)],
                         ids=["token_by_token", "whole", "twos", "mixed", "window_cut", "last_alone"])
def test_prompt_portions_and_decoding_agree_with_the_whole(dtype, portions):
    cfg = make_config(default_layers())
    W = random_weights(cfg, seed=9)
    tokens = torch.randint(0, cfg["vocab"], (70,), generator=torch.Generator().manual_seed(10)).tolist()
    want = _reference_logits(cfg, W, tokens)
    model = build_model(cfg, W, dtype, 70)
    got = _run_portions(model, tokens, portions)
    assert row_error(got, want).max() < _tol(dtype, cfg, W, tokens, want), row_error(got, want).max()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_fused_one_token_products_equal_the_unfused_step(dtype):
    """The decode step with the norm folded into hand-written products against the same step through library products
    and norm launches: same numbers up to summation order."""
    cfg = make_config(default_layers())
    W = random_weights(cfg, seed=21)
    tokens = torch.randint(0, cfg["vocab"], (40,), generator=torch.Generator().manual_seed(22)).tolist()
    outs = []
    for fused in (True, False):
        model = build_model(cfg, W, dtype, 40)
        model.fused_decode = fused
        assert model.kernels_per_token() == (3 + 4 * 7 + 2 * 6 if fused else 2 + 3 * 7 + 2 * 6)
        outs.append(_run_portions(model, tokens, (20,) + (1,) * 20))
    want = _reference_logits(cfg, W, tokens)
    assert row_error(outs[0], outs[1]).max() < (2e-5 if dtype == torch.float32 else 3e-2)
    assert row_error(outs[0], want).max() < _tol(dtype, cfg, W, tokens, want)


def test_one_token_product_kernel_alone():
    ops = _ops()
    from cold_compress_b200 import _lib
    g = torch.Generator().manual_seed(23)
    N, K, F = 37, 70, 29
    x, w, b = torch.randn(K, generator=g), torch.randn(N, K, generator=g) * 0.2, torch.randn(N, generator=g)
    nw, res, rw = torch.randn(K, generator=g) * 0.3, torch.randn(N, generator=g), torch.randn(N, generator=g) * 0.3
    xn = R.zero_centred_norm(x.double(), nw.double(), 1e-3)
    out = torch.empty(N, device=DEV)
    ops.seq_gemv(x.to(DEV), nw.to(DEV), w.to(DEV), b.to(DEV), None, None, out, _lib.GEMV_PLAIN, 1.0, 1e-3, 0.0, 0.0)
    assert (out.cpu().double() - (w.double() @ xn + b.double())).abs().max() < 1e-5
    ops.seq_gemv(x.to(DEV), None, w.to(DEV), None, res.to(DEV), rw.to(DEV), out, _lib.GEMV_RESIDUAL, 1.75, 1e-3, 0.0, 0.0)
    want = 1.75 * R.zero_centred_norm(res.double(), rw.double(), 1e-3) + w.double() @ x.double()
    assert (out.cpu().double() - want).abs().max() < 1e-5
    w2 = torch.randn(2 * F, K, generator=g)
    act = torch.empty(F, device=DEV)
    ops.seq_gemv(x.to(DEV), None, w2.to(DEV), None, None, None, act, _lib.GEMV_GLU, 1.0, 1e-3, 0.6, 1.702)
    gu = (w2.double() @ x.double())
    gate, up = gu[:F].clamp(max=0.6), gu[F:].clamp(-0.6, 0.6)
    assert (act.cpu().double() - gate * torch.sigmoid(1.702 * gate) * (up + 1)).abs().max() < 1e-5
    # bf16 weights and input, 16-byte rows
    K2 = 64
    xb, wb = torch.randn(K2, generator=g).to(torch.bfloat16), (torch.randn(N, K2, generator=g) * 0.2).to(torch.bfloat16)
    ops.seq_gemv(xb.to(DEV), None, wb.to(DEV), None, None, None, out, _lib.GEMV_PLAIN, 1.0, 1e-3, 0.0, 0.0)
    assert (out.cpu().double() - wb.double() @ xb.double()).abs().max() < 1e-5


def test_sequences_one_after_another_reuse_the_slots():
    """Three sequences of unequal length through one model, the caches given back in between: each equals itself
    alone.  The second is longer than the first, the third shorter, so rings and full caches are both re-filled and
    partly left empty."""
    from cold_compress_b200.generation_utils import reset_caches
    cfg = make_config(default_layers())
    W = random_weights(cfg, seed=11)
    g = torch.Generator().manual_seed(12)
    seqs = [torch.randint(0, cfg["vocab"], (n,), generator=g).tolist() for n in (45, 90, 13)]
    model = build_model(cfg, W, torch.float32, 90)
    for s, portions in zip(seqs, [(40, 1, 1, 1, 1, 1), (17, 60, 13), (13,)]):
        got = _run_portions(model, s, portions)
        want = _reference_logits(cfg, W, s)
        assert row_error(got, want).max() < fp32_tolerance(cfg, W, s, want)
        reset_caches(model)
        assert model.tok_embeddings.prev_token.item() == -1
        assert all(int(b.attention.kv_cache.cache_cts.item()) == 0 for b in model.layers)


def test_long_decoding_through_rings_and_splits():
    """300 prompt tokens, then 330 tokens one by one: the rings wrap many times and the global layers' decode kernel
    goes from two key splits to three."""
    cfg = make_config([window_layer(19), global_layer(), window_layer(260, dim=16, vdim=16), global_layer(heads=2, kv_heads=1, vdim=32)],
                      width=48, vocab=71)
    W = random_weights(cfg, seed=13)
    tokens = torch.randint(0, 71, (630,), generator=torch.Generator().manual_seed(14)).tolist()
    want = _reference_logits(cfg, W, tokens)
    model = build_model(cfg, W, torch.float32, 640)
    got = _run_portions(model, tokens, (300,) + (1,) * 330)
    assert row_error(got, want).max() < fp32_tolerance(cfg, W, tokens, want)


@pytest.mark.parametrize("layers,kw", [
    ([global_layer(heads=1, kv_heads=1, dim=8, vdim=8, every=1, ff=8)], dict(width=8, vocab=5, alpha=1.0, bigram=(1, 1, 1))),
    ([window_layer(2, heads=12, kv_heads=3, dim=130, vdim=70, ff=300, limit=0.3), global_layer(heads=12, kv_heads=12, dim=48, vdim=17, every=1000, coef=2.0, ff=0, v_mix=False)],
     dict(width=200, vocab=1000, alpha=0.5, eps=1e-2, scale=0.1, bigram=None)),
    ([global_layer(v_mix=False), window_layer(5), window_layer(6)], dict(width=33, vocab=17, bigram=(1009, 1000003, 999983))),
    ([global_layer(heads=34, kv_heads=2, dim=8, vdim=4, ff=30), window_layer(3, heads=17, kv_heads=1, dim=12, vdim=8, ff=0)],
     dict(width=51, vocab=77)),
], ids=["all_ones", "wide_heads_no_bigram", "odd_width_big_hash", "seventeen_query_heads_per_kv_head"])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_other_sizes(layers, kw, dtype):
    cfg = make_config(layers, **kw)
    W = random_weights(cfg, seed=15)
    tokens = torch.randint(0, cfg["vocab"], (29,), generator=torch.Generator().manual_seed(16)).tolist()
    want = _reference_logits(cfg, W, tokens)
    model = build_model(cfg, W, dtype, 32)
    got = _run_portions(model, tokens, (5, 1, 1, 20, 2))
    assert row_error(got, want).max() < _tol(dtype, cfg, W, tokens, want), row_error(got, want).max()


def test_second_norm_without_feed_forward():
    """A checkpoint that carries norm2 for a layer without feed-forward: the norm is applied to alpha * x, in prompt
    portions and in single-token steps (which then take the general step, not the fused products)."""
    cfg = make_config([global_layer(ff=0), window_layer(6), global_layer(ff=0, v_mix=False)], width=40, vocab=61)
    W = random_weights(cfg, seed=41)
    g = torch.Generator().manual_seed(42)
    W["l0.norm2"] = (torch.randn(40, generator=g) * 0.2).to(torch.bfloat16)
    tokens = torch.randint(0, 61, (24,), generator=g).tolist()
    want = _reference_logits(cfg, W, tokens)
    model = build_model(cfg, W, torch.float32, 24)
    assert model.layers[0].norm2 is not None and model.layers[2].norm2 is None and not model._fused_decode_fits()
    got = _run_portions(model, tokens, (10, 1, 1, 12))
    assert row_error(got, want).max() < fp32_tolerance(cfg, W, tokens, want)
    W.pop("l0.norm2")
    assert row_error(_reference_logits(cfg, W, tokens), want).max() > 1e-3   # the extra norm matters


def test_checkpoint_folder_generate_and_graphed_decoder(tmp_path):
    """From a checkpoint folder through load_model, setup_caches and generate(): greedy tokens equal the restatement's
    arg-max continuation, with the prompt whole or in portions, eager or graph-captured."""
    import json
    from pathlib import Path
    from cold_compress_b200.checkpoint import write_safetensors
    from cold_compress_b200.generation_utils import compile_funcs, generate, load_model, reset_caches, setup_caches
    cfg = make_config(default_layers())
    W = random_weights(cfg, seed=17)
    (tmp_path / "config.json").write_text(json.dumps(cfg))
    write_safetensors(tmp_path / "model.safetensors", W)
    prompt = torch.randint(0, cfg["vocab"], (33,), generator=torch.Generator().manual_seed(18)).tolist()
    new = 20
    # restatement: greedy continuation in float64 with the margin of every choice
    seq, margins = list(prompt), []
    for _ in range(new):
        lg = _reference_logits(cfg, W, seq)[-1]
        top = torch.topk(lg, 2).values
        margins.append((top[0] - top[1]).item())
        seq.append(int(lg.argmax()))
    model = load_model(Path(tmp_path), DEV, torch.float32, use_tp=False)
    setup_caches(model, None, DEV, len(prompt) + new, {})
    for compile_, chunk in ((False, None), (False, 7), (True, 2)):
        prefill, decode = compile_funcs(compile_)
        out, _, stats = generate(model, torch.tensor(prompt, dtype=torch.int32, device=DEV), prefill, decode,
                                 max_new_tokens=new, prefill_chunk=chunk)
        out = out.tolist()
        assert out[:len(prompt)] == prompt and len(out) == len(seq)
        for i, (a, b) in enumerate(zip(out[len(prompt):], seq[len(prompt):])):
            assert a == b or margins[i] < 1e-3, (compile_, chunk, i)
            if a != b:
                break
        assert stats["decode_tokens"] == new
        reset_caches(model)


def test_trace_replay_command(tmp_path):
    """bin/trace_run as a user runs it: a checkpoint folder, steps on standard input (a whole prompt, a prompt in
    portions with the last tokens alone, a second sequence after the first has ended), logits files and `done` lines."""
    import json
    import subprocess
    import sys
    from pathlib import Path
    import numpy as np
    from cold_compress_b200.checkpoint import write_safetensors
    root = Path(__file__).resolve().parent.parent
    cfg = make_config([global_layer(heads=6, kv_heads=3, dim=16, vdim=24, every=9), window_layer(13, heads=3, kv_heads=3, dim=24, vdim=24),
                       global_layer(heads=6, kv_heads=3, dim=16, vdim=24, ff=0), window_layer(50, heads=6, kv_heads=1, dim=8, vdim=72)],
                      width=88, vocab=301, alpha=3.0, bigram=(211, 13, 17))
    W = random_weights(cfg, seed=31)
    model_dir = tmp_path / "ckpt"
    model_dir.mkdir()
    (model_dir / "config.json").write_text(json.dumps(cfg))
    write_safetensors(model_dir / "model.safetensors", W)
    g = torch.Generator().manual_seed(32)
    a = torch.randint(0, 301, (75,), generator=g).tolist()
    b = torch.randint(0, 301, (41,), generator=g).tolist()
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": a[:30], "want": [0, 29]}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": a[30:32], "want": []}], "end": []},
             {"step": 2, "entries": [{"id": "a", "tokens": a[32:73], "want": [5, 40]}], "end": []},
             {"step": 3, "entries": [{"id": "a", "tokens": a[73:74], "want": [0]}], "end": []},
             {"step": 4, "entries": [{"id": "a", "tokens": a[74:75], "want": [0]}], "end": ["a"]},
             {"step": 5, "entries": [{"id": "b", "tokens": b, "want": [0, 20, 40]}], "end": ["b"]}]
    want = {0: [0, 29], 2: [37, 72], 3: [73], 4: [74]}
    la, lb = _reference_logits(cfg, W, a), _reference_logits(cfg, W, b)
    for dtype, tol in (("float32", 2e-4), ("bfloat16", BF16_TOL)):
        out = tmp_path / ("out_" + dtype)
        r = subprocess.run([sys.executable, str(root / "bin" / "trace_run"), "--model", str(model_dir), "--dtype", dtype,
                            "--out", str(out), "--max-tokens", "75"], input="\n".join(json.dumps(s) for s in steps) + "\n",
                           capture_output=True, text=True, timeout=600)
        assert r.returncode == 0, r.stderr[-2000:]
        assert [ln for ln in r.stdout.splitlines() if ln.startswith("done")] == [f"done {i}" for i in range(6)]
        assert not (out / "1.f32").exists()
        for step, rows in want.items():
            got = torch.from_numpy(np.fromfile(out / f"{step}.f32", dtype="<f4").reshape(len(rows), -1).copy())
            assert row_error(got, la[rows]).max() < tol, (dtype, step)
        got = torch.from_numpy(np.fromfile(out / "5.f32", dtype="<f4").reshape(3, -1).copy())
        assert row_error(got, lb[[0, 20, 40]]).max() < tol
