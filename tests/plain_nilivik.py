"""Plain, slow implementation of the Nilivik decoder: the oracle of its tests.

Whole sequences only, no cache, no batching, one function per mechanism, on the CPU in the dtype of
the tensors handed in (float64 for the oracle). It shares no code with the package under test: it
reads ``config.json`` and ``model.safetensors`` itself.

The model in this file's notation (x: residual stream [T, W], t: position, counted from 0):

* embedding      x_t = E[token_t] * s_e + pe(t), pe(t)[2i] = sin(t * b^(-2i/W)), pe(t)[2i+1] = cos(same), b = 10000
* scalar norm    n(x) = g * x / sqrt(mean(x^2) + eps), g one number
* layer          x += mixer(n1(x)); x += ff(n2(x)) (the second line only if the layer has a feed-forward)
* loop           layers [start, stop) run ``times`` times with the same weights; before pass p > 0 the
                 embedding output is added to x, and before every pass the row p of the step table
* parallel mixer c_l * left(a) + c_r * right(a)
* left           grouped-query attention without rotation; score_ij = q_i.k_j * s - r1 * ln(1 + r2 * (i - j));
                 i sees j <= i inside its own chunk of C positions; softmax whose denominator also holds
                 exp(sink); heads * sigmoid(Wg a), then Wo
* right          q, k, v = silu(W a); per head S_t = d * S_(t-1) + k_t v_t^T, o_t = S_t^T q_t; all heads
                 together through a weighted RMS norm, * sigmoid(Wg a), then Wo
* feed-forward   Wd f(Wu a), f(z) = ap z^2 + z/2 for z > 0, an (e^z - 1 - z) + z/2 otherwise,
                 ap = softplus(p), an = 1/2 + softplus(q)
* output         cap * tanh(head . n(x) / cap)
"""
import json
import math
import os

import torch
import torch.nn.functional as F
from safetensors import safe_open

SINUSOID_BASE = 10000.0


def read_model(folder, dtype=torch.float64):
    with open(os.path.join(folder, "config.json")) as f:
        cfg = json.load(f)
    tensors = {}
    with safe_open(os.path.join(folder, "model.safetensors"), framework="pt") as f:
        for k in f.keys():
            t = f.get_tensor(k)
            tensors[k] = t.to(dtype) if t.dtype.is_floating_point else t
    return cfg, tensors


def sinusoid(positions, width, dtype):
    """[len(positions), width]: sin at even places, cos at odd ones, one frequency per pair."""
    p = torch.as_tensor(positions, dtype=torch.float64)[:, None]
    i = torch.arange(width // 2, dtype=torch.float64)[None, :]
    ang = p * SINUSOID_BASE ** (-2.0 * i / width)
    out = torch.zeros(p.shape[0], width, dtype=torch.float64)
    out[:, 0::2] = torch.sin(ang)
    out[:, 1::2] = torch.cos(ang)
    return out.to(dtype)


def embedding(tokens, table, scale, first_position=0):
    x = table[torch.as_tensor(tokens, dtype=torch.long)] * scale
    return x + sinusoid(range(first_position, first_position + len(tokens)), table.shape[1], x.dtype)


def scalar_norm(x, g, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * g


def weighted_norm(x, w, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * w


def chunk_mask(T, chunk):
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    return (j <= i) & (i // chunk == j // chunk)


def attention_core(q, k, v, scale, chunk=None, r1=None, r2=None, sink=None, window=None, first_position=0):
    """q [T, H, D], k [T, G, D], v [T, G, Dv] of one whole sequence -> heads [T, H, Dv]. Every option
    is written out separately: mask (causal, chunk, window), distance bias, sink."""
    T, H = q.shape[0], q.shape[1]
    G = k.shape[1]
    pos = torch.arange(first_position, first_position + T)
    i, j = pos[:, None], pos[None, :]
    see = j <= i
    if chunk is not None:
        see = see & (i // chunk == j // chunk)
    if window is not None:
        see = see & (j > i - window)
    dist = (i - j).clamp(min=0).to(q.dtype)
    heads = []
    for h in range(H):
        g = h // (H // G)
        s = (q[:, h] @ k[:, g].T) * scale
        if r1 is not None:
            s = s - r1[h] * torch.log1p(r2[h] * dist)
        s = s.masked_fill(~see, -math.inf)
        top = s.max(-1, keepdim=True).values
        if sink is not None:
            top = torch.maximum(top, sink[h])
        e = torch.exp(s - top)
        den = e.sum(-1, keepdim=True)
        if sink is not None:
            den = den + torch.exp(sink[h] - top)
        heads.append((e / den) @ v[:, g])
    return torch.stack(heads, 1)


def left_attention(a, w, m):
    """``w``: the left mixer's tensors by short name; ``m``: its config. Returns [T, W]."""
    T = a.shape[0]
    H, G, D, Dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (a @ w["q"].T).view(T, H, D)
    k = (a @ w["k"].T).view(T, G, D)
    v = (a @ w["v"].T).view(T, G, Dv)
    chunk = m["mask"]["size"] if m.get("mask") else None
    heads = attention_core(q, k, v, m["scale"], chunk, w["r1"], w["r2"], w["sink"])
    o = heads.reshape(T, H * Dv) * torch.sigmoid(a @ w["g"].T)
    return o @ w["o"].T


def decay_recurrence(q, k, v, decay, state=None):
    """q, k [T, H, D], v [T, H, Dv] -> (o [T, H, Dv], last state [H, D, Dv]); token by token, exactly
    as the recurrence is written."""
    T, H, D = q.shape
    Dv = v.shape[2]
    S = torch.zeros(H, D, Dv, dtype=q.dtype) if state is None else state.clone()
    out = torch.zeros(T, H, Dv, dtype=q.dtype)
    for t in range(T):
        for h in range(H):
            S[h] = decay[h] * S[h] + torch.outer(k[t, h], v[t, h])
            out[t, h] = S[h].T @ q[t, h]
    return out, S


def right_recurrence(a, w, m, eps):
    T = a.shape[0]
    H, D, Dv = m["heads"], m["dim"], m["vdim"]
    decay = m["decay"] if isinstance(m["decay"], (list, tuple)) else [m["decay"]] * H
    q = F.silu(a @ w["q"].T).view(T, H, D)
    k = F.silu(a @ w["k"].T).view(T, H, D)
    v = F.silu(a @ w["v"].T).view(T, H, Dv)
    out, _ = decay_recurrence(q, k, v, decay)
    o = weighted_norm(out.reshape(T, H * Dv), w["norm"], eps) * torch.sigmoid(a @ w["g"].T)
    return o @ w["o"].T


def xielu(z, p, q):
    ap = F.softplus(p)
    an = 0.5 + F.softplus(q)
    return torch.where(z > 0, ap * z * z + 0.5 * z, an * (torch.expm1(z) - z) + 0.5 * z)


def dense_ff(a, w):
    return xielu(a @ w["up"].T, w["act"][0], w["act"][1]) @ w["down"].T


def _sub(tensors, prefix):
    return {k[len(prefix):]: v for k, v in tensors.items() if k.startswith(prefix)}


def layer(x, cfg, tensors, i):
    lc, eps = cfg["layers"][i], cfg["norm"]["eps"]
    if lc["type"] != "parallel":
        raise ValueError(f"layer type {lc['type']!r}")
    a = scalar_norm(x, tensors[f"l{i}.norm1"], eps)
    m = lc["mixer"]
    left = left_attention(a, _sub(tensors, f"l{i}.mix.left."), m["left"])
    right = right_recurrence(a, _sub(tensors, f"l{i}.mix.right."), m["right"], eps)
    x = x + m["left_scale"] * left + m["right_scale"] * right
    if lc.get("mlp") is not None:
        if lc["mlp"]["kind"] != "dense":
            raise ValueError(f"feed-forward kind {lc['mlp']['kind']!r}")
        x = x + dense_ff(scalar_norm(x, tensors[f"l{i}.norm2"], eps), _sub(tensors, f"l{i}.mlp."))
    return x


def layer_runs(cfg):
    """[(layer, pass number or None)] in running order; the pass number is set on the first layer of
    every pass of the loop."""
    n = len(cfg["layers"])
    loop = cfg.get("loop") or {"start": 0, "stop": 0, "times": 1}
    start, stop, times = loop["start"], loop["stop"], loop["times"]
    runs = [(i, None) for i in range(start)]
    for p in range(times):
        runs += [(i, p if i == start else None) for i in range(start, stop)]
    return runs + [(i, None) for i in range(stop, n)]


def forward(cfg, tensors, tokens, return_layers=False):
    """Logits [T, vocab] of one whole sequence (and, if asked, the stream after every layer run)."""
    x = e0 = embedding(tokens, tensors["embed"], cfg["embedding"]["scale"])
    seen = []
    for i, p in layer_runs(cfg):
        if p is not None:
            if p > 0:
                x = x + e0
            x = x + tensors["loop.step"][p]
        x = layer(x, cfg, tensors, i)
        seen.append(x)
    logits = scalar_norm(x, tensors["final.norm"], cfg["norm"]["eps"]) @ tensors["head"].T
    cap = cfg.get("logit_softcap")
    if cap:
        logits = cap * torch.tanh(logits / cap)
    return (logits, torch.stack(seen)) if return_layers else logits


def greedy(cfg, tensors, prompt, n):
    seq, out = list(prompt), []
    for _ in range(n):
        tok = int(forward(cfg, tensors, seq)[-1].argmax())
        out.append(tok)
        seq.append(tok)
    return out
