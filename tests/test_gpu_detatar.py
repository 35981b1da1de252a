"""GPU tests of the Detatar design: every mechanism's kernel against the plain restatement in detatar_reference.py
(float64, CPU, whole sequences), then the model through the runtime: layer by layer, prompt against token-by-token
decoding, prompt portions down to two tokens, state and caches that are given back and used again, one far key or
one old token that decides the output, long decoding, other sizes, greedy generation through generate() and the
graph-captured decoder, and the trace replay command."""
import json
import math

import pytest
import torch

import detatar_reference as R
from detatar_utils import (assert_rows_close, build_model, default_layers, dense, fp32_tolerance, latent_layer, make_config, moe, random_weights,
                           row_error, run_portions, wkv_layer)

pytestmark = pytest.mark.gpu
DEV = "cuda"
BF16_TOL = 6e-2
F64 = torch.float64


def _ops():
    from cold_compress_b200 import seq_ops
    return seq_ops


def _i32(*v):
    return torch.tensor(v, dtype=torch.int32, device=DEV)


def _tol(dtype, cfg, W, tokens, want):
    return BF16_TOL if dtype == torch.bfloat16 else fp32_tolerance(cfg, W, tokens, want)


# ----------------------------------------------------------------------------------------------- single mechanisms

@pytest.mark.parametrize("groups,E", [(1, 50), (3, 96), (5, 640)])
def test_gated_sum_and_group_norm_kernel(groups, E):
    ops = _ops()
    g = torch.Generator().manual_seed(groups)
    T = 7
    x, a, b = (torch.randn(T, E, generator=g) * 3 for _ in range(3))
    fused = torch.randn(T, 2 * E + 5, generator=g)                 # gate logits as column ranges of a wider product
    ba, bb, w = (torch.randn(E, generator=g) for _ in range(3))
    d = lambda t: t.double()
    xs = d(x) + d(a) * torch.sigmoid(d(fused[:, 3:3 + E]) + d(ba)) + d(b) * torch.sigmoid(d(fused[:, 3 + E:3 + 2 * E]) + d(bb))
    want = R.group_rms_norm(xs, d(w), groups, 1e-5)
    xd, fd = x.to(DEV), fused.to(DEV)
    h = torch.empty(T, E, device=DEV)
    ha = torch.empty(T, E, device=DEV, dtype=torch.bfloat16)
    ops.gated_group_norm(xd, w.to(DEV), groups, 1e-5, h, ha, a=a.to(DEV), ga=fd[:, 3:3 + E], ba=ba.to(DEV),
                         b=b.to(DEV), gb=fd[:, 3 + E:3 + 2 * E], bb=bb.to(DEV))
    assert (xd.cpu().double() - xs).abs().max() < 1e-5 and (h.cpu().double() - want).abs().max() < 2e-5
    assert torch.equal(ha, h.to(torch.bfloat16))
    # the sum alone, the norm alone, and a selection of rows
    x2 = x.to(DEV)
    ops.gated_group_norm(x2, None, 1, 0.0, a=a.to(DEV))
    assert (x2.cpu().double() - (d(x) + d(a))).abs().max() < 1e-5
    rows = torch.tensor([5, 0, 5], device=DEV)
    h3 = torch.empty(3, E, device=DEV)
    ops.gated_group_norm(x.to(DEV), w.to(DEV), groups, 1e-5, h3, None, rows=rows)
    assert (h3.cpu().double() - R.group_rms_norm(d(x), d(w), groups, 1e-5)[[5, 0, 5]]).abs().max() < 2e-5


def test_token_shift_kernel_carries_the_previous_row_across_portions():
    ops = _ops()
    g = torch.Generator().manual_seed(2)
    T, E, n = 19, 44, 5
    h, mu = torch.randn(T, E, generator=g), torch.rand(n, E, generator=g)
    want = torch.stack([R.shift_mix(h.double(), mu[s].double()) for s in range(n)])
    state = torch.zeros(E, device=DEV)
    got, at = [], 0
    for m in (1, 1, 2, 7, 1, 5, 2):
        out = torch.empty(n, m, E, device=DEV)
        outf = torch.empty(m, E, device=DEV)
        ops.token_shift(h[at:at + m].to(DEV).contiguous(), state, mu.to(DEV), out, outf)
        assert torch.equal(outf, out[0]) and torch.equal(state.cpu(), h[at + m - 1])
        got.append(out)
        at += m
    assert (torch.cat(got, 1).cpu().double() - want).abs().max() < 1e-6


@pytest.mark.parametrize("H,D,portions", [(1, 8, (40,)), (3, 33, (1, 2, 30, 1, 17)), (2, 64, (5,) + (1,) * 20), (2, 80, (33, 16, 1)),
                                              (1, 200, (20, 1, 19)), (1, 256, (9, 1, 12))])
def test_wkv_kernel_against_the_recurrence(H, D, portions):
    ops = _ops()
    g = torch.Generator().manual_seed(D)
    T = sum(portions)
    r, k, v = (torch.randn(T, H * D, generator=g) for _ in range(3))
    wraw = torch.randn(T, H * D, generator=g)
    w0 = torch.randn(H * D, generator=g) - 1.5
    u = torch.randn(H * D, generator=g) * 0.5
    w = torch.exp(-torch.exp(wraw.double() + w0.double()))
    sh = lambda t: t.double().reshape(T, H, D)
    want, S = R.wkv_recurrence(sh(r), sh(k), sh(v), sh(w), u.double().reshape(H, D))
    state = torch.zeros(H, D, D, device=DEV)
    got, at = [], 0
    for m in portions:
        o = torch.empty(m, H * D, device=DEV)
        sl = lambda t: t[at:at + m].to(DEV).contiguous()
        ops.wkv(sl(r), sl(k), sl(v), sl(wraw), w0.to(DEV), u.to(DEV), state, o, H, D)
        got.append(o)
        at += m
    scale = want.abs().max().item()
    assert (torch.cat(got).cpu().double().reshape(T, H, D) - want).abs().max() < 2e-5 * scale
    assert (state.cpu().double() - S).abs().max() < 2e-5 * S.abs().max()


@pytest.mark.parametrize("decode", [False, True])
def test_wkv_state_keeps_a_token_from_long_ago(decode):
    """Decays close to one and one loud token 600 steps back: the output at the end is that token's value, scaled
    by the decay it went through -- a state that was lost, reset or not carried would show."""
    ops = _ops()
    g = torch.Generator().manual_seed(3)
    H, D, T, far = 2, 32, 640, 37
    r, k, v = (torch.randn(T, H * D, generator=g) * 0.05 for _ in range(3))
    k[far] *= 400
    v[far] *= 400
    r[-1] *= 400
    wraw = torch.zeros(T, H * D)
    w0 = torch.full((H * D,), -7.0)
    u = torch.zeros(H * D)
    w = torch.exp(-torch.exp(wraw.double() + w0.double()))
    sh = lambda t: t.double().reshape(T, H, D)
    want, _ = R.wkv_recurrence(sh(r), sh(k), sh(v), sh(w), u.double().reshape(H, D))
    quiet_k = k.clone()
    quiet_k[far] /= 400
    without, _ = R.wkv_recurrence(sh(r), sh(quiet_k), sh(v), sh(w), u.double().reshape(H, D))
    assert (want[-1] - without[-1]).abs().max() > 10 * without[-1].abs().max()       # the far token decides
    state = torch.zeros(H, D, D, device=DEV)
    o = torch.empty(T, H * D, device=DEV)
    dv = lambda t: t.to(DEV).contiguous()
    if decode:
        n0 = 300
        ops.wkv(dv(r[:n0]), dv(k[:n0]), dv(v[:n0]), dv(wraw[:n0]), dv(w0), dv(u), state, o[:n0], H, D)
        for t in range(n0, T):
            ops.wkv(dv(r[t:t + 1]), dv(k[t:t + 1]), dv(v[t:t + 1]), dv(wraw[t:t + 1]), dv(w0), dv(u), state, o[t:t + 1], H, D)
    else:
        ops.wkv(dv(r), dv(k), dv(v), dv(wraw), dv(w0), dv(u), state, o, H, D)
    got = o.cpu().double().reshape(T, H, D)
    assert (got[-1] - want[-1]).abs().max() < 1e-4 * want[-1].abs().max()
    assert (got - want).abs().max() < 1e-4 * want.abs().max()


def test_head_norm_gate_and_gated_unit_kernels():
    ops = _ops()
    g = torch.Generator().manual_seed(4)
    T, H, D = 6, 3, 20
    o, nw = torch.randn(T, H * D, generator=g) * 4, torch.randn(H * D, generator=g)
    wide = torch.randn(T, H * D + 9, generator=g)
    od = o.double().reshape(T, H, D)
    want = (od / torch.sqrt((od * od).mean(-1, keepdim=True) + 1e-5)).reshape(T, H * D) * nw.double() * R.silu(wide[:, 9:].double())
    out = torch.empty(T, H * D, device=DEV)
    ops.head_norm_gate(o.to(DEV), wide.to(DEV)[:, 9:], nw.to(DEV), out, H, D, 1e-5)
    assert (out.cpu().double() - want).abs().max() < 1e-5
    from cold_compress_b200 import _lib
    src = torch.randn(T, 50, generator=g) * 2
    for kind, fn in ((_lib.ACT_GELU_TANH, R.gelu_tanh), (_lib.ACT_SILU, R.silu), (_lib.ACT_TANH, torch.tanh)):
        out = torch.empty(T, 20, device=DEV)
        ops.gated_unit(src.to(DEV), 3, 27, out, kind)
        assert (out.cpu().double() - fn(src[:, 3:23].double()) * src[:, 27:47].double()).abs().max() < 1e-5
        ops.gated_unit(src.to(DEV), 3, -1, out, kind)
        assert (out.cpu().double() - fn(src[:, 3:23].double())).abs().max() < 1e-5


def test_latent_rows_and_rotation_far_positions():
    ops = _ops()
    g = torch.Generator().manual_seed(5)
    T, Q, C, Rd, dims, p0, base = 5, 12, 20, 10, 6, 90000, 5000.0
    src = torch.randn(T, 3 + Q + C + Rd + 2, generator=g)
    wq, wkv = torch.randn(Q, generator=g), torch.randn(C, generator=g)
    inv = torch.pow(torch.tensor(base, dtype=F64), -2.0 * torch.arange(dims // 2, dtype=F64) / dims).float().to(DEV)
    cq = torch.empty(T, Q, device=DEV)
    krow = torch.empty(T, 1, C + Rd, device=DEV)
    vrow = torch.empty(T, 1, C, device=DEV)
    ops.latent_prepare(src.to(DEV), 3, Q, 3 + Q, C, Rd, dims, wq.to(DEV), wkv.to(DEV), inv, _i32(p0), cq, krow, vrow, 1e-5)
    pos = torch.arange(p0, p0 + T)
    s = src.double()
    assert (cq.cpu().double() - R.rms_norm(s[:, 3:3 + Q], wq.double(), 1e-5)).abs().max() < 1e-5
    c = R.rms_norm(s[:, 3 + Q:3 + Q + C], wkv.double(), 1e-5)
    kr = R.rope(s[:, 3 + Q + C:3 + Q + C + Rd], pos, base, dims)
    got = krow.cpu().double().reshape(T, C + Rd)
    # the angle is an fp32 product of a position near 1e5: allow its rounding
    assert (got[:, :C] - c).abs().max() < 1e-5 and (got[:, C:] - kr).abs().max() < 0.02
    assert torch.equal(vrow.reshape(T, C), krow.reshape(T, C + Rd)[:, :C])
    assert torch.equal(got[:, C + dims:], s[:, 3 + Q + C + dims:3 + Q + C + Rd].float().double())       # beyond the rotary dims: unchanged
    # heads of a fused query row: the same rotation on a segment of every head, at a small position exact to fp32
    H, hw, off = 3, 16, 6
    q = torch.randn(T, H * hw, generator=g)
    qd = q.to(DEV)
    tail = torch.zeros(T, H, 4 + Rd, device=DEV)
    ops.rope_heads(qd, _i32(11), inv, H, hw, off, Rd, dims, tail=tail, tail_off=4)
    want = q.double().reshape(T, H, hw).clone()
    want[..., off:] = R.rope(want[..., off:], torch.arange(11, 11 + T), base, dims)
    assert (qd.cpu().double().reshape(T, H, hw) - want).abs().max() < 1e-5
    assert torch.equal(tail[..., 4:].cpu(), qd.cpu().reshape(T, H, hw)[..., off:]) and float(tail[..., :4].abs().sum()) == 0


ROUTES = [(12, 4, 3, 4, 3), (8, 1, 1, 2, 0), (8, 8, 8, 8, 2), (40, 5, 2, 6, 10), (6, 3, 1, 1, 0), (3, 1, 1, 3, 1)]


@pytest.mark.parametrize("n,groups,keep,top,identity", ROUTES)
def test_router_kernel_against_the_rules(n, groups, keep, top, identity):
    ops = _ops()
    g = torch.Generator().manual_seed(n * 7 + top)
    T = 300
    wide = torch.randn(T, n + 4, generator=g) * 2
    corr = torch.randn(n, generator=g) * 0.2 - 0.3                 # negative choice scores: a masked group must not win by being 0
    r = {"experts": n - identity, "identity": identity, "top": top, "groups": {"count": groups, "keep": keep}}
    s = torch.softmax(wide[:, 2:2 + n].double(), -1)
    ids_w, w_w = R.route(wide[:, 2:2 + n].double(), torch.eye(n, dtype=F64), corr.double(), r)
    ids = torch.empty(T, top, dtype=torch.int32, device=DEV)
    wts = torch.empty(T, top, device=DEV)
    ops.moe_route(wide.to(DEV)[:, 2:2 + n], corr.to(DEV), ids, wts, groups, keep, top)
    ids, wts = ids.cpu().long(), wts.cpu().double()
    choice = s + corr.double()
    margin = torch.ones(T, dtype=torch.bool)      # rows whose choice does not hang on an fp32 rounding
    srt = choice.sort(-1, descending=True).values
    margin &= (srt[:, :-1] - srt[:, 1:]).min(-1).values > 1e-5 if n > 1 else margin
    same = (ids.sort(-1).values == ids_w.sort(-1).values).all(-1)
    assert same[margin].all() and margin.float().mean() > 0.8
    order = ids.argsort(-1), ids_w.argsort(-1)
    assert (wts.gather(1, order[0]) - w_w.gather(1, order[1]))[same].abs().max() < 1e-5
    assert (wts.sum(-1) - 1).abs().max() < 1e-5


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("T", [1, 3, 4, 5, 61])
def test_routed_experts_small_and_grouped_paths(T, dtype):
    """The mixture alone, below and above the size at which pairs are grouped by expert; both against the rules."""
    from cold_compress_b200 import _lib
    from cold_compress_b200.detatar import RoutedExperts
    g = torch.Generator().manual_seed(T)
    E, mlp = 48, moe(experts=5, identity=3, top=3, groups=2, keep=2, ff=16, shared=24)
    cfg = make_config([wkv_layer(mlp)], width=E)
    W = {k[len("l0.mlp."):]: v for k, v in random_weights(cfg, seed=T).items() if k.startswith("l0.mlp.")}
    m = RoutedExperts(E, 5, 3, 16, 3, 2, 2, 24, _lib.ACT_SILU, dtype)
    m.correction.data.copy_(W["correction"].float())
    m.w_gu.data.copy_(torch.stack([torch.cat([W[f"e{e}.gate"], W[f"e{e}.up"]]) for e in range(5)]).to(dtype))
    m.w_d.data.copy_(torch.stack([W[f"e{e}.down"] for e in range(5)]).to(dtype))
    m.w_shared_down.data.copy_(W["shared.down"].to(dtype))
    m = m.to(DEV)
    h = torch.randn(T, E, generator=g).to(torch.bfloat16)           # exactly representable in both dtypes
    rows = torch.cat([W["router"], W["shared.sg"], W["shared.gate"], W["shared.up"]]).double()
    hp = torch.cat([torch.zeros(T, 7, dtype=F64), h.double() @ rows.T], 1).float().to(DEV)
    got = m(hp, 7, h.float().to(DEV), h.to(dtype).to(DEV))
    want = R.moe(h.double(), {k: v.double() for k, v in W.items()}, mlp)
    err = (got.cpu().double() - want).abs().max() / want.abs().max()
    assert err < (3e-2 if dtype == torch.bfloat16 else 1e-5), err


def _latent_module(dtype, H=3, D=16, Rd=8, V=24, Q=20, C=40, E=64, base=10000.0, seed=0, scale=None):
    from cold_compress_b200.cache import get_cache_constructor
    from cold_compress_b200.detatar import LatentAttention
    cfg = make_config([latent_layer(None, heads=H, dim=D, rot_dim=Rd, vdim=V, q_rank=Q, kv_rank=C, base=base, scale=scale)], width=E)
    W = random_weights(cfg, seed=seed)
    P = {k[len("l0.mix."):]: v for k, v in W.items() if k.startswith("l0.mix.")}
    m = LatentAttention(E, H, D, Rd, V, Q, C, cfg["layers"][0]["mixer"]["scale"], base, Rd, 1e-5, dtype)
    rows = torch.cat([P["dq"], P["dkv"], P["g"]])
    m.w_in.data.zero_()
    m.w_in.data[:rows.shape[0]].copy_(rows.to(dtype))
    m.q_norm.data.copy_(P["dq.norm"].float())
    m.kv_norm.data.copy_(P["dkv.norm"].float())
    m.w_uq.data.copy_(P["uq"].to(dtype))
    m.w_ukv.data.copy_(torch.cat([P["uk"], P["uv"]]).to(dtype))
    m.w_uk_t.data.copy_(P["uk"].reshape(H, D, C).transpose(1, 2).to(dtype))
    m.w_o.data.copy_(P["o"].to(dtype))
    return m.to(DEV), {k: v.double() for k, v in P.items()}, cfg["layers"][0]["mixer"], get_cache_constructor("latent")[0]


@pytest.mark.parametrize("far", [0, 1, 255, 256, 640])
@pytest.mark.parametrize("mode", ["whole", "portions", "decode", "decode_expanded"])
def test_latent_attention_one_key_decides(far, mode):
    """The latents are normalised, so a key cannot be made loud by scaling its input.  Instead every earlier token is
    the same vector, the softmax is sharp (a large score scale), and the token at one position far back (also the very
    first one) is the candidate, out of a few dozen random vectors, whose key the last query likes best: one head's
    softmax then sits on that key, and a key that is dropped, misplaced or rotated by a wrong position would show.
    Whole prompt, portions, and single tokens through the absorbed and the expanded form."""
    T, E = 700, 64
    m, P, mix, ctor = _latent_module(torch.float32, scale=2.0)
    g = torch.Generator().manual_seed(far)
    hs = torch.randn(T, E, generator=g)
    hs[:-1] = torch.randn(E, generator=g)
    best, best_margin = None, -math.inf
    for cand in torch.randn(48, E, generator=g):
        trial = hs.clone()
        trial[far] = cand
        row = R.latent_scores(trial.double(), P, mix, 1e-5)[0][:, -1, :]
        others = row.clone()
        others[:, far] = -math.inf
        margin = (row[:, far] - others.max(-1).values).max().item()
        if margin > best_margin:
            best, best_margin = trial, margin
    want = R.latent_attention_mixer(best.double(), P, mix, 1e-5)
    plain = R.latent_attention_mixer(hs.double(), P, mix, 1e-5)
    assert best_margin > 20 and (plain[-1] - want[-1]).abs().max() > 0.2 * want[-1].abs().max()      # the far key decides
    with torch.device(DEV):
        cache = ctor(1, 1, m.row_width, torch.float32, v_head_dim=m.kv_rank, max_cache_length=T, max_seq_length=T)
    portions = {"whole": (T,), "portions": (3, 250, 2, 3, 380, 62), "decode": (650,) + (1,) * 50, "decode_expanded": (690,) + (1,) * 10}[mode]
    got, at = [], 0
    for n in portions:
        got.append(m(best[at:at + n].to(DEV).contiguous(), _i32(at), cache, one_token_kernel=mode != "decode_expanded"))
        at += n
    got = torch.cat(got).cpu().double()
    assert (got - want).abs().max() < 1e-4 * want.abs().max(), (got - want).abs().max() / want.abs().max()
    assert int(cache.cache_cts.item()) == T and torch.equal(cache.pos[0, 0].cpu(), torch.arange(T, dtype=torch.int32))


def test_latent_cache_rows_given_back_are_not_keys():
    """A second, shorter sequence after a longer one: the rows the first left behind must not be attended."""
    m, P, mix, ctor = _latent_module(torch.bfloat16, seed=3)
    g = torch.Generator().manual_seed(8)
    with torch.device(DEV):
        cache = ctor(1, 1, m.row_width, torch.bfloat16, v_head_dim=m.kv_rank, max_cache_length=64, max_seq_length=64)
    a, b = torch.randn(60, 64, generator=g).to(torch.bfloat16), torch.randn(21, 64, generator=g).to(torch.bfloat16)
    m(a.to(DEV), _i32(0), cache)
    cache.reset()
    got = [m(b[:9].to(DEV), _i32(0), cache), m(b[9:20].to(DEV), _i32(9), cache), m(b[20:].to(DEV), _i32(20), cache)]
    want = R.latent_attention_mixer(b.double(), P, mix, 1e-5)
    assert (torch.cat(got).cpu().double() - want).abs().max() < 3e-2 * want.abs().max()


# ----------------------------------------------------------------------------------------------- the model in the runtime

def _reference_logits(cfg, W, tokens, collect=None):
    return R.forward(cfg, W, tokens, collect)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_layers_one_by_one_and_logits(dtype):
    cfg = make_config(default_layers())
    W = random_weights(cfg, seed=5)
    tokens = torch.randint(0, cfg["vocab"], (41,), generator=torch.Generator().manual_seed(6)).tolist()
    ref_layers = []
    want = _reference_logits(cfg, W, tokens, ref_layers)
    model = build_model(cfg, W, dtype, 41)
    got_layers = []
    x = torch.tensor(tokens, dtype=torch.int32, device=DEV).view(1, -1)
    got = model(x, torch.arange(41, dtype=torch.int32, device=DEV), is_prefill=True, logits_at=torch.arange(41, device=DEV),
                collect=got_layers)[0]
    assert len(got_layers) == len(ref_layers) == len(cfg["layers"])
    for i, (a, b) in enumerate(zip(got_layers, ref_layers)):
        assert_rows_close((a.cpu().double() - b).abs().max(-1).values / b.abs().max(), dtype, 6e-2 if dtype == torch.bfloat16 else 2e-5, i)
    assert_rows_close(row_error(got, want), dtype, _tol(dtype, cfg, W, tokens, want))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("portions", [(1,) * 70, (70,), (2,) * 35, (3, 11, 1, 1, 37, 2, 2, 12, 1), (5, 4, 61), (69, 1)],
                         ids=["token_by_token", "whole", "twos", "mixed", "around_grouping", "last_alone"])
def test_prompt_portions_and_decoding_agree_with_the_whole(dtype, portions):
    cfg = make_config(default_layers())
    W = random_weights(cfg, seed=9)
    tokens = torch.randint(0, cfg["vocab"], (70,), generator=torch.Generator().manual_seed(10)).tolist()
    want = _reference_logits(cfg, W, tokens)
    model = build_model(cfg, W, dtype, 70)
    got = run_portions(model, tokens, portions)
    assert_rows_close(row_error(got, want), dtype, _tol(dtype, cfg, W, tokens, want))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_one_token_kernels_equal_the_portion_kernels(dtype):
    """A decode step through the one-token products and the absorbed attention against the same step through the
    kernels of a one-token prompt portion."""
    cfg = make_config(default_layers())
    W = random_weights(cfg, seed=15)
    tokens = torch.randint(0, cfg["vocab"], (50,), generator=torch.Generator().manual_seed(16)).tolist()
    outs = []
    for fused in (True, False):
        model = build_model(cfg, W, dtype, 50)
        model.fused_decode = fused
        outs.append(run_portions(model, tokens, (30,) + (1,) * 20))
    assert_rows_close(row_error(outs[0], outs[1]), dtype, BF16_TOL if dtype == torch.bfloat16 else 1e-5)
    assert model.kernels_per_token() > 0


def test_sequences_one_after_another_reuse_state_and_rows():
    """Three sequences of unequal length through one model, caches and state given back in between: each equals
    itself alone."""
    from cold_compress_b200.generation_utils import reset_caches
    cfg = make_config(default_layers())
    W = random_weights(cfg, seed=11)
    g = torch.Generator().manual_seed(12)
    seqs = [torch.randint(0, cfg["vocab"], (n,), generator=g).tolist() for n in (45, 90, 13)]
    model = build_model(cfg, W, torch.float32, 90)
    for s, portions in zip(seqs, [(40, 1, 1, 1, 1, 1), (17, 60, 13), (13,)]):
        got = run_portions(model, s, portions)
        want = _reference_logits(cfg, W, s)
        assert row_error(got, want).max() < fp32_tolerance(cfg, W, s, want)
        reset_caches(model)
        assert all(float(l.state.vectors.abs().sum()) == 0 and float(l.state.matrix.abs().sum()) == 0 for l in model.layers)
        assert all(int(l.kv_cache.cache_cts.item()) == 0 for l in model.layers if l.kv_cache is not None)


def test_long_decoding():
    """200 prompt tokens, then 330 tokens one by one: the one-token attention goes through several key splits and the
    recurrent state through hundreds of single steps."""
    cfg = make_config([wkv_layer(dense(40), heads=2, dim=16), latent_layer(moe(experts=4, identity=0, top=2, groups=2, keep=1, ff=16, shared=0)),
                       latent_layer(None, heads=2, dim=8, rot_dim=8, vdim=16, kv_rank=24)], width=48, vocab=71, groups=1)
    W = random_weights(cfg, seed=13)
    tokens = torch.randint(0, 71, (530,), generator=torch.Generator().manual_seed(14)).tolist()
    want = _reference_logits(cfg, W, tokens)
    model = build_model(cfg, W, torch.float32, 540)
    got = run_portions(model, tokens, (200,) + (1,) * 330)
    assert row_error(got, want).max() < fp32_tolerance(cfg, W, tokens, want)


OTHER = [
    # every size that can be one is one; no identity experts, no shared expert, one group
    ([wkv_layer(moe(experts=2, identity=0, top=1, groups=1, keep=1, ff=1, shared=0), heads=1, dim=1),
      latent_layer(dense(1), heads=1, dim=1, rot_dim=2, vdim=1, q_rank=1, kv_rank=1)], dict(width=4, vocab=5, groups=1)),
    # latent rows wider than the one-token attention kernel takes, and more heads than it holds: the expanded form decodes
    ([latent_layer(dense(48), heads=2, dim=8, rot_dim=8, vdim=8, kv_rank=264), latent_layer(None, heads=17, dim=8, rot_dim=4, vdim=8, kv_rank=16)],
     dict(width=64, vocab=90, groups=4)),
    # rotary dims below the rotated width, unrotated width zero-free odd sizes, head size of the recurrence not a multiple of 32
    ([latent_layer(moe(experts=3, identity=1, top=2, groups=2, keep=1, ff=10, shared=6), heads=5, dim=6, rot_dim=10, vdim=14, q_rank=9, kv_rank=18, dims=4, base=300.0),
      wkv_layer(None, heads=3, dim=17), wkv_layer(dense(30), heads=1, dim=70), wkv_layer(None, heads=3, dim=17, weights_of=1)],
     dict(width=70, vocab=60, groups=7, scale=0.7)),
    # only dense feed-forwards and only recurrent mixers
    ([wkv_layer(dense(64), heads=4, dim=32), wkv_layer(dense(64), heads=4, dim=32, weights_of=0)], dict(width=128, vocab=33, groups=2)),
]


@pytest.mark.parametrize("layers,kw", OTHER, ids=["ones", "wide_latent_many_heads", "odd_sizes", "recurrent_only"])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_other_sizes(layers, kw, dtype):
    cfg = make_config(layers, **kw)
    W = random_weights(cfg, seed=21, decay_rank=3)
    tokens = torch.randint(0, cfg["vocab"], (48,), generator=torch.Generator().manual_seed(22)).tolist()
    want = _reference_logits(cfg, W, tokens)
    model = build_model(cfg, W, dtype, 48)
    got = run_portions(model, tokens, (5, 2, 30, 1, 1, 6, 1, 1, 1))
    assert_rows_close(row_error(got, want), dtype, _tol(dtype, cfg, W, tokens, want))


def test_checkpoint_folder_generate_and_graphed_decoder(tmp_path):
    """From a checkpoint folder through load_model, setup_caches and generate(): greedy tokens equal the restatement's
    arg-max continuation, with the prompt whole or in portions, eager or graph-captured."""
    from pathlib import Path
    from cold_compress_b200.checkpoint import write_safetensors
    from cold_compress_b200.generation_utils import compile_funcs, generate, load_model, reset_caches, setup_caches
    cfg = make_config(default_layers())
    W = random_weights(cfg, seed=17)
    (tmp_path / "config.json").write_text(json.dumps(cfg))
    write_safetensors(tmp_path / "model.safetensors", W)
    prompt = torch.randint(0, cfg["vocab"], (33,), generator=torch.Generator().manual_seed(18)).tolist()
    new = 20
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
    """bin/trace_run as a user runs it: a checkpoint folder, steps on standard input (a whole prompt, portions with the
    last tokens alone, a second sequence after the first has ended), logits files and `done` lines."""
    import subprocess
    import sys
    from pathlib import Path
    import numpy as np
    from cold_compress_b200.checkpoint import write_safetensors
    root = Path(__file__).resolve().parent.parent
    cfg = make_config([latent_layer(dense(40)), wkv_layer(moe()), latent_layer(dense(40), weights_of=0), wkv_layer(None, heads=2, dim=12)],
                      width=72, vocab=211, groups=2)
    W = random_weights(cfg, seed=31)
    model_dir = tmp_path / "ckpt"
    model_dir.mkdir()
    (model_dir / "config.json").write_text(json.dumps(cfg))
    write_safetensors(model_dir / "model.safetensors", W)
    g = torch.Generator().manual_seed(32)
    a = torch.randint(0, 211, (75,), generator=g).tolist()
    b = torch.randint(0, 211, (41,), generator=g).tolist()
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": a[:30], "want": [0, 29]}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": a[30:32], "want": []}], "end": []},
             {"step": 2, "entries": [{"id": "a", "tokens": a[32:73], "want": [5, 40]}], "end": []},
             {"step": 3, "entries": [{"id": "a", "tokens": a[73:74], "want": [0]}], "end": []},
             {"step": 4, "entries": [{"id": "a", "tokens": a[74:75], "want": [0]}], "end": ["a"]},
             {"step": 5, "entries": [{"id": "b", "tokens": b, "want": [0, 20, 40]}], "end": ["b"]}]
    want = {0: [0, 29], 2: [37, 72], 3: [73], 4: [74]}
    la, lb = _reference_logits(cfg, W, a), _reference_logits(cfg, W, b)
    for dtype, tol in (("float32", 2e-4), ("bfloat16", 2 * BF16_TOL)):
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
