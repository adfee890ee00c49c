"""A plain, slow Ditalorn: one function per mechanism, written from the architecture's equations in double precision
with torch on the CPU. It shares no code with the engine and is what the engine's kernels are compared with.

Notation: x [T, W] is a sequence's residual stream (rows are positions 0..T-1), `cfg` the dictionary of config.json,
`w` a dictionary name -> tensor (any floating dtype; everything is widened to float64).

    x = embed[token] * embedding.scale + pos[position]
    layer i:   x = x + n(mixer(n(x, norm1)), norm1b);   x = x + n(experts(n(x, norm2)), norm2b)      n(v, name) = rms(v) * (1 + w[name])
    logits = embed n(x, final.norm)
"""
from __future__ import annotations

import math

import torch

F64 = torch.float64


def d(t):
    return t.to(F64)


# ------------------------------------------------------------------------------------------ small pieces
def rms_unit(x, eps):
    """x over the root of (its mean square + eps), along the last axis."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def norm_offset(x, weight, eps):
    """RMS norm whose stored weight lies around zero."""
    return rms_unit(x, eps) * (1.0 + d(weight))


def norm_plain(x, weight, eps):
    return rms_unit(x, eps) * d(weight)


def silu(z):
    return z * torch.sigmoid(z)


def causal_conv(u, taps_w):
    """y[t, c] = sum_j taps_w[c, j] * u[t - K + 1 + j, c]; rows before the sequence's start are zero. taps_w [C, K]."""
    T, C = u.shape
    K = taps_w.shape[1]
    padded = torch.cat([torch.zeros((K - 1, C), dtype=u.dtype), u], 0)
    y = torch.zeros_like(u)
    for j in range(K):
        y = y + d(taps_w)[:, j] * padded[j:j + T]
    return y


def embed(tokens, cfg, w):
    T = len(tokens)
    return d(w["embed"])[torch.tensor(tokens, dtype=torch.long)] * float((cfg.get("embedding") or {}).get("scale", 1.0)) + d(w["pos"])[:T]


# ------------------------------------------------------------------------------------------ latent attention with a window
def windowed_softmax(q, k, v, scale, window):
    """q, k [T, H, dim], v [T, H, vdim]: position i sees j with 0 <= i - j < window (window None: every j <= i); softmax over those."""
    T = q.shape[0]
    s = torch.einsum("ihd,jhd->hij", q, k) * scale
    dist = torch.arange(T).view(T, 1) - torch.arange(T).view(1, T)
    seen = (dist >= 0) if window is None else (dist >= 0) & (dist < window)
    a = torch.softmax(s.masked_fill(~seen, -math.inf), dim=-1)
    return torch.einsum("hij,jhv->ihv", a, v)


def latent_attention(h, m, w, p, eps):
    """Queries through a normed latent; keys and values of every head as maps of one normed latent a token; a position sees itself
    and the mask.size - 1 positions before it; softmax; every head's output times the sigmoid of its gate."""
    T = h.shape[0]
    H, dim, vdim = int(m["heads"]), int(m["dim"]), int(m["vdim"])
    cq = norm_plain(h @ d(w[p + ".dq"]).T, w[p + ".dq.norm"], eps)
    q = (cq @ d(w[p + ".uq"]).T).view(T, H, dim)
    c = norm_plain(h @ d(w[p + ".dkv"]).T, w[p + ".dkv.norm"], eps)
    k = (c @ d(w[p + ".uk"]).T).view(T, H, dim)
    v = (c @ d(w[p + ".uv"]).T).view(T, H, vdim)
    mask = m.get("mask") or {}
    o = windowed_softmax(q, k, v, float(m["scale"]), None if mask.get("size") is None else int(mask["size"]))
    gate = torch.sigmoid(h @ d(w[p + ".g"]).T)             # [T, H]
    o = o * gate.unsqueeze(-1)
    return o.reshape(T, H * vdim) @ d(w[p + ".o"]).T


# ------------------------------------------------------------------------------------------ attention with sigmoid weights
def query_temperature(T, qt):
    """1 + coef * ln(floor((p + 1) / every) + 1) for p = 0..T-1."""
    p = torch.arange(T, dtype=torch.long)
    return 1.0 + float(qt["coef"]) * torch.log((torch.div(p + 1, int(qt["every"]), rounding_mode="floor") + 1).to(F64))


def distance_bias(T, r1, r2):
    """[H, T, T]: r1_h * ln(1 + r2_h * (i - j)) for j <= i (zero elsewhere)."""
    i = torch.arange(T).view(T, 1)
    j = torch.arange(T).view(1, T)
    dist = (i - j).clamp(min=0).to(F64)
    return d(r1).view(-1, 1, 1) * torch.log1p(d(r2).view(-1, 1, 1) * dist)


def sigmoid_weights(q, k, v, scale, r1, r2, pb):
    """q [T, H, dim], k [T, G, dim], v [T, G, vdim] -> [T, H, vdim]: o_i = sum_{j <= i} sigmoid(q_i . k_j * scale - bias(i - j) + pb) v_j."""
    T, H = q.shape[0], q.shape[1]
    rep = H // k.shape[1]
    k, v = k.repeat_interleave(rep, dim=1), v.repeat_interleave(rep, dim=1)
    s = torch.einsum("ihd,jhd->hij", q, k) * scale
    if r1 is not None:
        s = s - distance_bias(T, r1, r2)
    if pb is not None:
        s = s + d(pb).view(H, 1, 1)
    a = torch.sigmoid(s) * torch.tril(torch.ones((T, T), dtype=F64))
    return torch.einsum("hij,jhv->ihv", a, v)


def sigmoid_attention(h, m, w, p, eps):
    """Grouped heads; biased projections; a short causal convolution on every channel of q, k, v; q times a temperature of its
    position; values divided by their root mean square per head; score minus a bias that grows with the distance; the weight of
    a key is the sigmoid of its score plus a number per head, and weights are not normalised."""
    T = h.shape[0]
    H, G, dim, vdim = int(m["heads"]), int(m.get("kv_heads") or m["heads"]), int(m["dim"]), int(m.get("vdim") or m["dim"])

    def proj(name):
        u = h @ d(w[f"{p}.{name}"]).T + d(w[f"{p}.{name}.b"])
        return causal_conv(u, w[f"{p}.{name}.conv"]) if m.get("conv") else u

    q = proj("q").view(T, H, dim)
    if m.get("q_temp"):
        q = q * query_temperature(T, m["q_temp"]).view(T, 1, 1)
    k = proj("k").view(T, G, dim)
    v = rms_unit(proj("v").view(T, G, vdim), eps)
    o = sigmoid_weights(q, k, v, float(m["scale"]), w[p + ".r1"], w[p + ".r2"], w[p + ".pb"])
    return o.reshape(T, H * vdim) @ d(w[p + ".o"]).T + d(w[p + ".o.b"])


# ------------------------------------------------------------------------------------------ experts
def route(h, f, w, p):
    """(chosen experts [T, top], their weights [T, top]). Choice scores are sigmoid(logit) + correction; a group's score is the sum of its
    two largest choice scores; only the experts of the best groups.keep groups can be chosen; the weights are the plain sigmoids."""
    r = f["router"]
    g = r.get("groups") or {}
    return choose(torch.sigmoid(h @ d(w[p + ".router"]).T), d(w[p + ".correction"]), int(r["top"]), int(g.get("count") or 1), int(g.get("keep") or g.get("count") or 1))


def choose(s, correction, top, n_groups, keep):
    """s [T, E] scores in (0, 1) -> (chosen experts [T, top], their weights [T, top])."""
    T, E = s.shape
    choice = s + correction
    per = E // n_groups
    grouped = choice.view(T, n_groups, per)
    gscore = grouped.topk(min(2, per), dim=-1).values.sum(-1)
    kept = gscore.topk(keep, dim=-1).indices
    allowed = torch.zeros((T, n_groups), dtype=torch.bool)
    allowed.scatter_(1, kept, True)
    masked = choice.masked_fill(~allowed.unsqueeze(-1).expand(T, n_groups, per).reshape(T, E), -math.inf)
    idx = masked.topk(top, dim=-1).indices
    return idx, s.gather(1, idx)


def expert(h, w, p):
    return (silu(h @ d(w[p + ".gate"]).T) * (h @ d(w[p + ".up"]).T)) @ d(w[p + ".down"]).T


def experts(h, f, w, p):
    idx, wt = route(h, f, w, p)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e, a in zip(idx[t].tolist(), wt[t].tolist()):
            out[t] = out[t] + a * expert(h[t:t + 1], w, f"{p}.e{e}")[0]
    return out


# ------------------------------------------------------------------------------------------ the model
MIXERS = {"latent_attention": latent_attention, "attention": sigmoid_attention}


def hidden_states(tokens, cfg, w):
    """The residual stream after the embedding and after every layer: a list of [T, W]."""
    eps = float(cfg["norm"]["eps"])
    x = embed(tokens, cfg, w)
    out = [x.clone()]
    for i, l in enumerate(cfg["layers"]):
        p = f"l{i}"
        a = MIXERS[l["type"]](norm_offset(x, w[p + ".norm1"], eps), l["mixer"], w, p + ".mix", eps)
        x = x + norm_offset(a, w[p + ".norm1b"], eps)
        if l.get("mlp") is not None:
            f = experts(norm_offset(x, w[p + ".norm2"], eps), l["mlp"], w, p + ".mlp")
            x = x + norm_offset(f, w[p + ".norm2b"], eps)
        out.append(x.clone())
    return out


def logits(tokens, cfg, w):
    x = hidden_states(tokens, cfg, w)[-1]
    return norm_offset(x, w["final.norm"], float(cfg["norm"]["eps"])) @ d(w["embed"]).T


def greedy(prompt, n, cfg, w):
    """n tokens, each the largest logit after everything before it (the lowest id on a tie)."""
    toks = list(prompt)
    for _ in range(n):
        toks.append(int(torch.argmax(logits(toks, cfg, w)[-1])))
    return toks[len(prompt):]
