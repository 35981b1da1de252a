"""Small random Tidelorn checkpoints for the tests: configurations, weights under the checkpoint's tensor names, and
error measures.  The sizes here are the tests' own."""
from __future__ import annotations

import copy

import torch


def global_layer(heads=4, kv_heads=2, dim=24, vdim=16, coef=0.4, every=5, v_mix=True, ff=80, limit=0.8, scale=None):
    return {"type": "attention",
            "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale or dim ** -0.5,
                      "q_temp": {"coef": coef, "every": every}, "v_mix": v_mix},
            "mlp": {"kind": "dense", "ff": ff, "limit": limit} if ff else None}


def window_layer(window, heads=4, kv_heads=2, dim=40, vdim=16, v_mix=True, ff=56, limit=2.5, scale=None):
    return {"type": "attention_2",
            "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale or dim ** -0.5,
                      "mask": {"size": window}, "v_mix": v_mix},
            "mlp": {"kind": "dense", "ff": ff, "limit": limit} if ff else None}


def make_config(layers, width=72, vocab=131, alpha=1.7, eps=1e-5, scale=5.5, bigram=(53, 5, 3)):
    cfg = {"architecture": "Tidelorn", "vocab": vocab, "width": width, "postln_alpha": alpha, "norm": {"eps": eps},
           "embedding": {"scale": scale}, "layers": copy.deepcopy(layers)}
    if bigram:
        cfg["embedding"]["bigram"] = {"buckets": bigram[0], "mul_prev": bigram[1], "mul_cur": bigram[2]}
    return cfg


def default_layers():
    """Window first (so the first value-mixing layer is a sliding one), two global layers with different head
    splits, a layer without value mixing, a layer without feed-forward, a one-token window."""
    return [window_layer(11), global_layer(), global_layer(heads=8, kv_heads=4, dim=16, vdim=8, every=3),
            window_layer(4, v_mix=False, dim=24, vdim=24, heads=2, kv_heads=2), global_layer(v_mix=False, ff=0),
            window_layer(1, ff=40), window_layer(37, heads=6, kv_heads=2, dim=20)]


def random_weights(cfg, seed=0):
    """bf16 tensors under the checkpoint's names; gains, sinks and mixing coefficients away from their neutral values."""
    g = torch.Generator().manual_seed(seed)
    E, V = cfg["width"], cfg["vocab"]

    def rnd(*shape, s=1.0):
        return (torch.randn(*shape, generator=g) * s).to(torch.bfloat16)

    W = {"embed": rnd(V, E, s=0.3), "final.norm": rnd(E, s=0.2), "head": rnd(V, E, s=E ** -0.5)}
    big = cfg["embedding"].get("bigram")
    if big:
        W["bigram"] = rnd(big["buckets"] + 1, E, s=0.5)
    for i, layer in enumerate(cfg["layers"]):
        m, p = layer["mixer"], f"l{i}."
        H, G, Dk, Dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
        W[p + "mix.q"], W[p + "mix.k"], W[p + "mix.v"] = rnd(H * Dk, E, s=E ** -0.5), rnd(G * Dk, E, s=E ** -0.5), rnd(G * Dv, E, s=E ** -0.5)
        W[p + "mix.o"] = rnd(E, H * Dv, s=(H * Dv) ** -0.5 * 2.0)
        W[p + "mix.vmix"] = (torch.rand((), generator=g) * 0.6 + 0.2).to(torch.bfloat16)
        W[p + "norm1"] = rnd(E, s=0.2)
        if layer["type"] == "attention":
            W[p + "mix.q.b"], W[p + "mix.k.b"], W[p + "mix.v.b"] = rnd(H * Dk, s=0.3), rnd(G * Dk, s=0.3), rnd(G * Dv, s=0.3)
            W[p + "mix.sink"] = rnd(H, s=1.5)
        if layer.get("mlp"):
            F = layer["mlp"]["ff"]
            W[p + "mlp.gate"], W[p + "mlp.up"] = rnd(F, E, s=E ** -0.5 * 1.5), rnd(F, E, s=E ** -0.5 * 1.5)
            W[p + "mlp.down"] = rnd(E, F, s=F ** -0.5 * 2.0)
            W[p + "norm2"] = rnd(E, s=0.2)
    return W


def as_double(W):
    return {k: (v.double() if v.is_floating_point() else v) for k, v in W.items()}


def row_error(got, want):
    """Per row: rms of the difference with its mean removed, over the rms of the wanted rows (all rows pooled)."""
    got, want = got.double().cpu(), want.double().cpu()
    d = got - want
    d = d - d.mean(-1, keepdim=True)
    ref = (want - want.mean(-1, keepdim=True)).pow(2).mean().sqrt()
    return d.pow(2).mean(-1).sqrt() / ref


def build_model(cfg, W, dtype, max_seq_length, device="cuda"):
    from cold_compress_b200.generation_utils import setup_caches
    from cold_compress_b200.tidelorn import TidelornTransformer
    model = TidelornTransformer.from_config(cfg, dtype)
    model.load_tensors(W)
    model = model.to(device).eval()
    setup_caches(model, None, device, max_seq_length, {})
    return model


def fp32_tolerance(cfg, W, tokens, want):
    """Three times the row error that fp32 rounding alone causes in the restatement itself (float32 against float64
    on the CPU): the bar for the fp32 kernels.  These small random models amplify rounding more than a trained one."""
    import tidelorn_reference as R
    W32 = {k: (v.float() if v.is_floating_point() else v) for k, v in W.items()}
    return max(3.0 * row_error(R.forward(tokens, W32, cfg), want).max().item(), 5e-6)
