"""Pibulix restated plainly: one slow function per mechanism, float64 throughout, straight from the
equations. Shares no code with the package; the tests compare the package with this.

Notation: T tokens of one sequence, positions 0..T-1; W width; H heads, G key/value heads, D key size,
V value size; weights are [out, in] and act as x @ W.T.
"""
import math

import torch

F = torch.float64


def rms(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def norm_one_plus(x, w, eps):
    """RMS norm whose stored weight sits around zero: the gain is 1 + w."""
    return rms(x, eps) * (1.0 + w)


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def silu(z):
    return z * torch.sigmoid(z)


def short_conv(u, w):
    """u [T, C], w [C, taps]: y_t = sum_j w[:, j] * u_(t - taps + 1 + j), zeros before the start."""
    T, C = u.shape
    taps = w.shape[1]
    pad = torch.cat([torch.zeros(taps - 1, C, dtype=u.dtype), u], 0)
    y = torch.zeros_like(u)
    for j in range(taps):
        y = y + pad[j:j + T] * w[:, j]
    return y


def rotate_partial(x, pos, dims, base):
    """x [T, heads, D]: the first ``dims`` coordinates of each head turn, coordinate i with i + dims/2,
    by the angle pos * base^(-2i/dims); the rest pass."""
    half = dims // 2
    f = torch.tensor([base ** (-2.0 * i / dims) for i in range(half)], dtype=F)
    a = pos.to(F)[:, None] * f[None, :]
    c, s = torch.cos(a)[:, None, :], torch.sin(a)[:, None, :]
    u, v = x[..., :half], x[..., half:dims]
    return torch.cat([u * c - v * s, v * c + u * s, x[..., dims:]], -1)


def visible(i, j, size, keep_first):
    return j <= i and (i - j < size or j < keep_first)


def attention_core(q, k, v, scale, size, keep_first, softcap, pos0=0):
    """q [T, H, D], k [T, G, D], v [T, G, V] at positions pos0.. -> [T, H, V]: capped scores, the window with its
    kept first tokens, and a softmax whose denominator has one added."""
    T, H, _ = q.shape
    G, V = k.shape[1], v.shape[2]
    out = torch.zeros(T, H, V, dtype=F)
    see = torch.tensor([[visible(pos0 + i, pos0 + j, size if size else 1 << 60, keep_first) for j in range(T)] for i in range(T)])
    for hd in range(H):
        g = hd // (H // G)
        s = (q[:, hd] @ k[:, g].T) * scale
        if softcap:
            s = softcap * torch.tanh(s / softcap)
        e = torch.where(see, torch.exp(s), torch.zeros_like(s))
        out[:, hd] = (e / (1.0 + e.sum(-1, keepdim=True))) @ v[:, g]
    return out


def attention_mixer(h, p, m, eps, pos0=0):
    """h [T, W]; p: tensors q, k, v, o, q.norm, k.norm, q.conv, k.conv, v.conv; m: the mixer's config."""
    T = h.shape[0]
    H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q, k, v = h @ p["q"].T, h @ p["k"].T, h @ p["v"].T
    if "q.conv" in p:
        q, k, v = short_conv(q, p["q.conv"]), short_conv(k, p["k.conv"]), short_conv(v, p["v.conv"])
    q, k, v = q.view(T, H, D), k.view(T, G, D), v.view(T, G, V)
    q = rms(q, eps) * p["q.norm"]
    k = rms(k, eps) * p["k.norm"]
    pos = torch.arange(pos0, pos0 + T)
    if m.get("rot") and m["rot"]["dims"]:
        q = rotate_partial(q, pos, m["rot"]["dims"], m["rot"]["base"])
        k = rotate_partial(k, pos, m["rot"]["dims"], m["rot"]["base"])
    mask = m.get("mask") or {}
    out = attention_core(q, k, v, m["scale"], mask.get("size"), mask.get("keep_first", 0), m.get("softcap") or None, pos0)
    return out.reshape(T, H * V) @ p["o"].T


def gla_recurrence(q, k, v, alpha, S=None):
    """q, k, alpha [T, H, D], v [T, H, V]: S_t = diag(alpha_t) S_(t-1) + k_t v_t^T, o_t = S_t^T q_t."""
    T, H, D = q.shape
    V = v.shape[-1]
    S = torch.zeros(H, D, V, dtype=F) if S is None else S.clone()
    o = torch.zeros(T, H, V, dtype=F)
    for t in range(T):
        S = alpha[t][:, :, None] * S + k[t][:, :, None] * v[t][:, None, :]
        o[t] = torch.einsum("hdv,hd->hv", S, q[t])
    return o, S


def gla_mixer(h, p, m, eps):
    T = h.shape[0]
    H, D, V = m["heads"], m["dim"], m["vdim"]
    q = (h @ p["q"].T * D ** -0.5).view(T, H, D)
    k = (h @ p["k"].T).view(T, H, D)
    v = (h @ p["v"].T).view(T, H, V)
    z = (h @ p["a1"].T) @ p["a2"].T + p["a2.b"]
    alpha = torch.sigmoid(z).pow(1.0 / m["tau"]).view(T, H, D)
    o, _ = gla_recurrence(q, k, v, alpha)
    o = rms(o, eps) * p["norm"]
    return (o.reshape(T, H * V) * silu(h @ p["g"].T)) @ p["o"].T


def dense_ff(h, p):
    return (gelu_tanh(h @ p["gate"].T) * (h @ p["up"].T)) @ p["down"].T


def expert(h, gate, up, down):
    return (silu(h @ gate.T) * (h @ up.T)) @ down.T


def route(z, correction, top, groups, keep, scale):
    """z [T, E] router logits -> chosen experts [T, top] and their weights."""
    s = torch.sigmoid(z)
    c = s + correction
    T, E = z.shape
    per = E // groups
    gs = c.view(T, groups, per).topk(min(2, per), -1).values.sum(-1)
    best = gs.topk(keep, -1).indices
    allowed = torch.zeros(T, groups, dtype=torch.bool)
    allowed.scatter_(1, best, True)
    c = torch.where(allowed[:, :, None].expand(T, groups, per).reshape(T, E), c, torch.full_like(c, -math.inf))
    idx = c.topk(top, -1).indices
    w = s.gather(1, idx)
    return idx, w / (w.sum(-1, keepdim=True) + 1e-20) * scale


def moe_ff(h, p, m):
    r = m["router"]
    idx, w = route(h @ p["router"].T, p["correction"], r["top"], r["groups"]["count"], r["groups"]["keep"], r["scale"])
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for j in range(r["top"]):
            e = int(idx[t, j])
            out[t] += w[t, j] * expert(h[t:t + 1], p[f"e{e}.gate"], p[f"e{e}.up"], p[f"e{e}.down"])[0]
    if "shared.gate" not in p:
        return out
    sh = expert(h, p["shared.gate"], p["shared.up"], p["shared.down"])
    return out + sh * torch.sigmoid(h @ p["shared.sg"].T)


def sub(tensors, prefix):
    return {k[len(prefix):]: v for k, v in tensors.items() if k.startswith(prefix)}


def forward(config, tensors, tokens, layers_out=None):
    """Logits [T, vocab] of one sequence run whole. ``tensors``: name -> float64 tensor."""
    eps, alpha = config["norm"]["eps"], config["postln_alpha"]
    x = tensors["embed"][torch.as_tensor(tokens)]
    for i, lc in enumerate(config["layers"]):
        src = lc.get("weights_of", i)
        pre = f"l{src}."
        mix = sub(tensors, pre + "mix.")
        if lc["type"] == "attention":
            d = attention_mixer(x, mix, lc["mixer"], eps)
        elif lc["type"] == "gla":
            d = gla_mixer(x, mix, lc["mixer"], eps)
        else:
            raise ValueError(lc["type"])
        x = norm_one_plus(alpha * x + d, tensors[pre + "norm1"], eps)
        if lc.get("mlp") is not None:
            mlp = sub(tensors, pre + "mlp.")
            d = dense_ff(x, mlp) if lc["mlp"]["kind"] == "dense" else moe_ff(x, mlp, lc["mlp"])
            x = norm_one_plus(alpha * x + d, tensors[pre + "norm2"], eps)
        if layers_out is not None:
            layers_out.append(x.clone())
    x = norm_one_plus(x, tensors["final.norm"], eps)
    return x @ tensors["head"].T


def read_model(folder):
    """config.json as a dict and every tensor of model.safetensors in float64."""
    import json
    import os

    from safetensors import safe_open

    with open(os.path.join(folder, "config.json")) as f:
        config = json.load(f)
    tensors = {}
    with safe_open(os.path.join(folder, "model.safetensors"), "pt") as f:
        for k in f.keys():
            tensors[k] = f.get_tensor(k).to(F)
    return config, tensors
