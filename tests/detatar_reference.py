"""Plain restatement of the Detatar design for the tests: whole sequences, dense masks, one function per mechanism, in
the dtype of the tensors it is given (float64 for the oracle, float32 to measure what rounding alone does).  Nothing
here is shared with the package."""
import math
import torch



def group_rms_norm(x, w, groups, eps):
    T, E = x.shape
    xg = x.reshape(T, groups, E // groups)
    xg = xg / torch.sqrt((xg * xg).mean(-1, keepdim=True) + eps)
    return xg.reshape(T, E) * w


def rms_norm(x, w, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * w


def shift_mix(h, mu):
    """h + (previous h - h) * mu, previous of the first token = 0."""
    prev = torch.cat([torch.zeros_like(h[:1]), h[:-1]], 0)
    return h + (prev - h) * mu


def gelu_tanh(z):
    return 0.5 * z * (1 + torch.tanh(math.sqrt(2 / math.pi) * (z + 0.044715 * z ** 3)))


def silu(z):
    return z * torch.sigmoid(z)


def glu(h, gate, up, down, act):
    return (act(h @ gate.T) * (h @ up.T)) @ down.T


def rope(v, pos, base, dims):
    """v [T, ..., D]: rotate-half pairs (i, i + dims/2) of the first `dims` entries."""
    half = dims // 2
    f = base ** (-2.0 * torch.arange(half, dtype=v.dtype) / dims)
    ang = pos.to(v.dtype)[:, None] * f
    shape = [v.shape[0]] + [1] * (v.dim() - 2) + [half]
    c, s = torch.cos(ang).reshape(shape), torch.sin(ang).reshape(shape)
    a, b = v[..., :half], v[..., half:dims]
    return torch.cat([a * c - b * s, b * c + a * s, v[..., dims:]], -1)


def wkv_recurrence(r, k, v, w, u, S=None):
    """r, k, v, w [T, H, D], u [H, D] -> out [T, H, D], final state [H, D, D] (key channel x value channel)."""
    T, H, D = r.shape
    S = torch.zeros(H, D, D, dtype=r.dtype) if S is None else S.clone()
    out = torch.zeros(T, H, D, dtype=r.dtype)
    for t in range(T):
        kv = k[t][:, :, None] * v[t][:, None, :]
        out[t] = torch.einsum("hi,hij->hj", r[t], S + u[:, :, None] * kv)
        S = w[t][:, :, None] * S + kv
    return out, S


def wkv_mixer(h, P, m, eps):
    T, E = h.shape
    H, D = m["heads"], m["dim"]
    mix = {s: shift_mix(h, P["mu." + s]) for s in "rkvgw"}
    r = (mix["r"] @ P["r"].T).reshape(T, H, D)
    k = (mix["k"] @ P["k"].T).reshape(T, H, D)
    v = (mix["v"] @ P["v"].T).reshape(T, H, D)
    gate = silu(mix["g"] @ P["g"].T)
    w = torch.exp(-torch.exp(torch.tanh(mix["w"] @ P["w1"].T) @ P["w2"].T + P["w0"])).reshape(T, H, D)
    out, _ = wkv_recurrence(r, k, v, w, P["u"].reshape(H, D))
    out = out / torch.sqrt((out * out).mean(-1, keepdim=True) + eps)
    return (out.reshape(T, H * D) * P["norm"] * gate) @ P["o"].T


def latent_scores(h, P, m, eps):
    """-> scaled, causally masked scores [H, T, T], the latents c [T, kv_rank] and the output gate logits."""
    T, E = h.shape
    H, D, R, C = m["heads"], m["dim"], m["rot_dim"], m["kv_rank"]
    pos = torch.arange(T)
    cq = rms_norm(h @ P["dq"].T, P["dq.norm"], eps)
    q = (cq @ P["uq"].T).reshape(T, H, D + R)
    kv = h @ P["dkv"].T
    c = rms_norm(kv[:, :C], P["dkv.norm"], eps)
    kr = rope(kv[:, C:], pos, m["rot"]["base"], m["rot"]["dims"])
    qr = rope(q[..., D:], pos, m["rot"]["base"], m["rot"]["dims"])
    ku = (c @ P["uk"].T).reshape(T, H, D)
    s = (torch.einsum("ihd,jhd->hij", q[..., :D], ku) + torch.einsum("ihd,jd->hij", qr, kr)) * m["scale"]
    return s.masked_fill(pos[None, :, None] < pos[None, None, :], -math.inf), c


def latent_attention_mixer(h, P, m, eps):
    T, E = h.shape
    H, V = m["heads"], m["vdim"]
    s, c = latent_scores(h, P, m, eps)
    val = (c @ P["uv"].T).reshape(T, H, V)
    o = torch.einsum("hij,jhv->ihv", torch.softmax(s, -1), val)
    o = o * torch.sigmoid(h @ P["g"].T)[:, :, None]
    return o.reshape(T, H * V) @ P["o"].T


def route(h, router, correction, r):
    """-> chosen ids [T, top], weights [T, top] over experts + identity experts."""
    n = r["experts"] + r.get("identity", 0)
    s = torch.softmax(h @ router.T, -1)
    choice = s + correction
    G, keep = r["groups"]["count"], r["groups"]["keep"]
    gs = choice.reshape(-1, G, n // G).max(-1).values
    best = gs.topk(keep, -1).indices
    allowed = torch.zeros_like(gs, dtype=torch.bool).scatter_(1, best, True)
    allowed = allowed[:, :, None].expand(-1, -1, n // G).reshape(-1, n)
    ids = choice.masked_fill(~allowed, -math.inf).topk(r["top"], -1).indices
    w = s.gather(1, ids)
    return ids, w / (w.sum(-1, keepdim=True) + 1e-20)


def moe(h, P, mlp):
    r = mlp["router"]
    ids, w = route(h, P["router"], P["correction"], r)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e, we in zip(ids[t].tolist(), w[t]):
            if e >= r["experts"]:
                out[t] += we * h[t]
            else:
                out[t] += we * glu(h[t:t + 1], P[f"e{e}.gate"], P[f"e{e}.up"], P[f"e{e}.down"], silu)[0]
    if mlp.get("shared"):
        sh = glu(h, P["shared.gate"], P["shared.up"], P["shared.down"], silu)
        out = out + sh * torch.sigmoid(h @ P["shared.sg"].T)
    return out


def sub(tensors, prefix, F):
    return {k[len(prefix):]: v.to(F) for k, v in tensors.items() if k.startswith(prefix)}


def forward(cfg, tensors, tokens, collect=None, F=torch.float64):
    """tokens: list of ids -> logits [T, vocab] in dtype F."""
    eps, groups = cfg["norm"]["eps"], cfg["norm"].get("groups", 1)
    x = tensors["embed"].to(F)[torch.tensor(tokens)] * cfg["embedding"]["scale"]
    for i, layer in enumerate(cfg["layers"]):
        p = "l%d." % layer.get("weights_of", i)
        L = sub(tensors, p, F)
        h = group_rms_norm(x, L["norm1"], groups, eps)
        hs = shift_mix(h, L["shift"])
        M = sub(tensors, p + "mix.", F)
        if layer["type"] == "wkv":
            a = wkv_mixer(hs, M, layer["mixer"], eps)
        elif layer["type"] == "latent_attention":
            a = latent_attention_mixer(hs, M, layer["mixer"], eps)
        else:
            raise ValueError(layer["type"])
        y = a * torch.sigmoid(h @ L["rg1"].T + L["rg1.b"])
        mlp = layer.get("mlp")
        if mlp:
            Q = sub(tensors, p + "mlp.", F)
            f = glu(h, Q["gate"], Q["up"], Q["down"], gelu_tanh) if mlp["kind"] == "dense" else moe(h, Q, mlp)
            y = y + f * torch.sigmoid(h @ L["rg2"].T + L["rg2.b"])
        x = x + y
        if collect is not None:
            collect.append(x.clone())
    x = group_rms_norm(x, tensors["final.norm"].to(F), groups, eps)
    return x @ tensors["head"].to(F).T
