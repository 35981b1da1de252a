"""Small random Detatar checkpoints for the tests: configurations, weights under the checkpoint's tensor names, and
error measures.  The sizes here are the tests' own."""
from __future__ import annotations

import copy

import torch

from tidelorn_utils import row_error  # noqa: F401  (same error measure for both designs)


def dense(ff=72):
    return {"kind": "dense", "ff": ff}


def moe(experts=6, identity=2, top=3, groups=4, keep=2, ff=24, shared=40):
    cfg = {"kind": "moe", "expert": {"ff": ff},
           "router": {"experts": experts, "identity": identity, "top": top, "groups": {"count": groups, "keep": keep}}}
    if shared:
        cfg["shared"] = {"ff": shared}
    return cfg


def latent_layer(mlp, heads=3, dim=16, rot_dim=8, vdim=24, q_rank=20, kv_rank=40, base=10000.0, dims=None, scale=None, weights_of=None):
    layer = {"type": "latent_attention",
             "mixer": {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "q_rank": q_rank, "kv_rank": kv_rank,
                       "scale": scale or (dim + rot_dim) ** -0.5, "rot": {"base": base, "dims": rot_dim if dims is None else dims}},
             "mlp": mlp}
    if weights_of is not None:
        layer["weights_of"] = weights_of
    return layer


def wkv_layer(mlp, heads=3, dim=24, weights_of=None):
    layer = {"type": "wkv", "mixer": {"heads": heads, "dim": dim}, "mlp": mlp}
    if weights_of is not None:
        layer["weights_of"] = weights_of
    return layer


def make_config(layers, width=96, vocab=151, groups=3, eps=1e-5, scale=2.5):
    return {"architecture": "Detatar", "vocab": vocab, "width": width, "norm": {"eps": eps, "groups": groups},
            "embedding": {"scale": scale}, "layers": copy.deepcopy(layers)}


def default_layers():
    """Both mixers with both feed-forwards, a layer without feed-forward, and two layers that run an earlier layer's
    weights on a state and cache of their own."""
    m = moe()
    return [wkv_layer(dense()), latent_layer(m), latent_layer(dense(56), heads=2, dim=8, rot_dim=16, vdim=8, dims=12),
            wkv_layer(m, heads=2, dim=40), latent_layer(None), latent_layer(m, weights_of=1), wkv_layer(dense(), weights_of=0)]


def random_weights(cfg, seed=0, decay_rank=6):
    """bf16 tensors under the checkpoint's names; gains, biases and mixing coefficients away from their neutral values."""
    g = torch.Generator().manual_seed(seed)
    E, V = cfg["width"], cfg["vocab"]

    def rnd(*shape, s=1.0, mean=0.0):
        return (torch.randn(*shape, generator=g) * s + mean).to(torch.bfloat16)

    def uni(*shape):
        return torch.rand(*shape, generator=g).to(torch.bfloat16)

    def glu(p, F):
        W[p + "gate"], W[p + "up"], W[p + "down"] = rnd(F, E, s=E ** -0.5 * 1.5), rnd(F, E, s=E ** -0.5 * 1.5), rnd(E, F, s=F ** -0.5 * 2.0)

    W = {"embed": rnd(V, E, s=0.4), "final.norm": rnd(E, s=0.2, mean=1.0), "head": rnd(V, E, s=E ** -0.5)}
    for i, layer in enumerate(cfg["layers"]):
        if layer.get("weights_of") is not None:
            continue
        m, p = layer["mixer"], f"l{i}."
        W[p + "norm1"], W[p + "shift"] = rnd(E, s=0.2, mean=1.0), uni(E)
        W[p + "rg1"], W[p + "rg1.b"] = rnd(E, E, s=E ** -0.5), rnd(E, s=0.5)
        if layer["type"] == "wkv":
            hd = m["heads"] * m["dim"]
            for s in "rkvgw":
                W[p + "mix.mu." + s] = uni(E)
            for s in "rkvg":
                W[p + "mix." + s] = rnd(hd, E, s=E ** -0.5)
            W[p + "mix.w1"], W[p + "mix.w2"] = rnd(decay_rank, E, s=E ** -0.5), rnd(hd, decay_rank, s=0.5)
            W[p + "mix.w0"], W[p + "mix.u"] = rnd(hd, s=1.0, mean=-2.0), rnd(m["heads"], m["dim"], s=0.5)
            W[p + "mix.norm"], W[p + "mix.o"] = rnd(hd, s=0.2, mean=1.0), rnd(E, hd, s=hd ** -0.5 * 2.0)
        else:
            H, D, R, Vd, C, Q = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"], m["q_rank"]
            W[p + "mix.dq"], W[p + "mix.dq.norm"] = rnd(Q, E, s=E ** -0.5), rnd(Q, s=0.2, mean=1.0)
            W[p + "mix.uq"] = rnd(H * (D + R), Q, s=Q ** -0.5 * 2.0)
            W[p + "mix.dkv"], W[p + "mix.dkv.norm"] = rnd(C + R, E, s=E ** -0.5 * 2.0), rnd(C, s=0.2, mean=1.0)
            W[p + "mix.uk"], W[p + "mix.uv"] = rnd(H * D, C, s=C ** -0.5 * 2.0), rnd(H * Vd, C, s=C ** -0.5)
            W[p + "mix.g"], W[p + "mix.o"] = rnd(H, E, s=E ** -0.5 * 2.0), rnd(E, H * Vd, s=(H * Vd) ** -0.5 * 2.0)
        mlp = layer.get("mlp")
        if not mlp:
            continue
        W[p + "rg2"], W[p + "rg2.b"] = rnd(E, E, s=E ** -0.5), rnd(E, s=0.5)
        if mlp["kind"] == "dense":
            glu(p + "mlp.", mlp["ff"])
        else:
            r = mlp["router"]
            n = r["experts"] + r.get("identity", 0)
            # scores well apart, corrections of both signs (choice scores may be negative)
            W[p + "mlp.router"], W[p + "mlp.correction"] = rnd(n, E, s=E ** -0.5 * 3.0), rnd(n, s=0.15, mean=-0.05)
            for e in range(r["experts"]):
                glu(f"{p}mlp.e{e}.", mlp["expert"]["ff"])
            if mlp.get("shared"):
                glu(p + "mlp.shared.", mlp["shared"]["ff"])
                W[p + "mlp.shared.sg"] = rnd(1, E, s=E ** -0.5 * 2.0)
    return W


def build_model(cfg, W, dtype, max_seq_length, device="cuda"):
    from cold_compress_b200.detatar import DetatarTransformer
    from cold_compress_b200.generation_utils import setup_caches
    model = DetatarTransformer.from_config(cfg, dtype)
    model.load_tensors(W)
    model = model.to(device).eval()
    setup_caches(model, None, device, max_seq_length, {})
    return model


def fp32_tolerance(cfg, W, tokens, want):
    """Three times the row error that fp32 rounding alone causes in the restatement itself (float32 against float64
    on the CPU): the bar for the fp32 kernels."""
    import detatar_reference as R
    return max(3.0 * row_error(R.forward(cfg, W, tokens, F=torch.float32), want).max().item(), 5e-6)


def run_portions(model, tokens, portions, device="cuda"):
    """Feeds `tokens` in consecutive portions through the runtime's step function; logits of every position."""
    from cold_compress_b200.generation_utils import model_step
    assert sum(portions) == len(tokens)
    out, at = [], 0
    for n in portions:
        x = torch.tensor(tokens[at:at + n], dtype=torch.int32, device=device).view(1, -1)
        ip = torch.arange(at, at + n, dtype=torch.int32, device=device)
        lg = model_step(model, x, ip, is_prefill=not (n == 1 and at > 0), logits_at=torch.arange(n, device=device))
        out.append(lg[0].float())
        at += n
    return torch.cat(out, 0)


def assert_rows_close(err, dtype, tol, what=""):
    """err: one error per position.  fp32: every position within `tol`.  bf16: the median within a third of `tol` and
    at most one position in twenty (or one) beyond it -- with random weights a few tokens sit where two experts'
    choice scores differ by less than a bf16 rounding of the router's input, and either choice is a correct bf16 result."""
    err = torch.as_tensor(err).double().reshape(-1)
    if dtype == torch.bfloat16:
        over = int((err > tol).sum())
        assert over <= max(1, len(err) // 20) and err.median() < tol / 3, (what, over, err.median().item(), err.max().item())
    else:
        assert err.max() < tol, (what, err.max().item(), int(err.argmax()))
