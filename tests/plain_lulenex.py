"""A plain, slow Lulenex: one function per mechanism, written from the architecture's equations in double precision with torch
on the CPU. It shares no code with the engine and is what the engine's kernels are compared with.

Notation: x [T, W] is one sequence's residual stream (rows are positions 0..T-1), `cfg` the dictionary of config.json, `w` a
dictionary name -> tensor (any floating dtype; everything is widened to float64).

    x0 = embed[tokens]
    the layers `loop.start .. loop.stop - 1` are run `loop.times` times in a row; before the first of them, in every pass t:
               x = loop.in [x ; x0] + loop.step[t]
    layer:     h = g1 * rms(x);  h_t <- h_t + (h_(t-1) - h_t) * shift  (h_(-1) = 0);  x = x + mixer(h)
               x = x + down xielu(up (g2 * rms(x)))                                    (a layer may have no feed-forward)
    logits = head (g * rms(x))
"""
from __future__ import annotations

import math

import torch

F64 = torch.float64


def d(t):
    return t.to(F64)


# ------------------------------------------------------------------------------------------ small pieces
def rms_unit(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def scalar_norm(x, g, eps):
    """An RMS norm whose weight is one number for all channels."""
    return rms_unit(x, eps) * d(g).reshape(())


def silu(z):
    return z * torch.sigmoid(z)


def softplus(z):
    return torch.log1p(torch.exp(-z.abs())) + torch.clamp(z, min=0)


def token_shift(h, mix):
    """Row t becomes h_t + (h_(t-1) - h_t) * mix, with the rows as they were before the replacement and zeros before row 0."""
    before = torch.cat([torch.zeros_like(h[:1]), h[:-1]], 0)
    return h + (before - h) * d(mix)


def xielu(z, pq):
    """z > 0: softplus(p) z^2 + z / 2;  z <= 0: (1/2 + softplus(q)) (exp(z) - 1 - z) + z / 2."""
    p, q = softplus(d(pq)[0]), softplus(d(pq)[1])
    pos = p * z * z + 0.5 * z
    neg = (0.5 + q) * (torch.expm1(torch.clamp(z, max=0.0)) - z) + 0.5 * z
    return torch.where(z > 0, pos, neg)


def dense_ff(h, w, p):
    return xielu(h @ d(w[f"{p}.up"]).T, w[f"{p}.act"]) @ d(w[f"{p}.down"]).T


# ------------------------------------------------------------------------------------------ rotation
def rotate(x, positions, dims, base):
    """x [T, heads, dim]: entry i of the first `dims` is turned together with entry i + dims/2 by the angle position * base^(-2i/dims)."""
    half = dims // 2
    if half == 0:
        return x
    f = torch.tensor([base ** (-2.0 * i / dims) for i in range(half)], dtype=F64)
    a = d(positions)[:, None, None] * f
    u, v = x[..., :half], x[..., half:dims]
    return torch.cat([u * torch.cos(a) - v * torch.sin(a), v * torch.cos(a) + u * torch.sin(a), x[..., dims:]], -1)


# ------------------------------------------------------------------------------------------ the left mixer: chunked attention with a sink
def sink_softmax_in_blocks(q, k, v, pos, scale, size, sink):
    """q [T, H, D], k and v [T, G, D] at positions pos -> [T, H, D]: position i weighs the positions j <= i of its own block of `size`
    positions (i // size == j // size) by exp(q_i . k_j * scale), and the denominator also holds exp(sink) of the head."""
    T, H, D = q.shape
    G = k.shape[1]
    out = torch.zeros((T, H, v.shape[2]), dtype=F64)
    i, j = pos[:, None], pos[None, :]
    seen = (j <= i) & (i // size == j // size)
    for a in range(H):
        b = a // (H // G)
        s = ((q[:, a] @ k[:, b].T) * scale).masked_fill(~seen, -math.inf)
        top = torch.maximum(s.max(-1, keepdim=True).values, sink[a])
        e = torch.exp(s - top)
        out[:, a] = (e / (e.sum(-1, keepdim=True) + torch.exp(sink[a] - top))) @ v[:, b]
    return out


def chunked_attention(h, w, p, m, eps):
    """Grouped-query attention whose values are its keys as projected; scores of rotated, unit-normed q and k; a position sees
    the earlier positions of its own chunk of `mask.size`; the softmax's denominator also holds exp(sink) per head; every head's
    output is gated by one sigmoid."""
    T = h.shape[0]
    H, G, D = int(m["heads"]), int(m["kv_heads"]), int(m["dim"])
    size, scale = int(m["mask"]["size"]), float(m["scale"])
    q = (h @ d(w[f"{p}.q"]).T + d(w[f"{p}.q.b"])).view(T, H, D)
    k = (h @ d(w[f"{p}.k"]).T + d(w[f"{p}.k.b"])).view(T, G, D)
    v = k
    pos = torch.arange(T)
    rot = m["rot"]
    q = rms_unit(rotate(q, pos, int(rot["dims"]), float(rot["base"])), eps)
    k = rms_unit(rotate(k, pos, int(rot["dims"]), float(rot["base"])), eps)
    gate = torch.sigmoid(h @ d(w[f"{p}.g"]).T)                      # [T, H]
    out = sink_softmax_in_blocks(q, k, v, pos, scale, size, d(w[f"{p}.sink"])) * gate[:, :, None]
    return out.reshape(T, H * D) @ d(w[f"{p}.o"]).T + d(w[f"{p}.o.b"])


# ------------------------------------------------------------------------------------------ the right mixer: a linear recurrence with a fixed decay
def decayed_linear_attention(h, w, p, m, eps):
    """Per head S_t = decay S_(t-1) + k_t v_t^T, o_t = S_t^T q_t with q, k, v = silu of their projections; all heads' o normed together,
    gated elementwise by a sigmoid, projected."""
    T = h.shape[0]
    H, D, V = int(m["heads"]), int(m["dim"]), int(m["vdim"])
    q = silu(h @ d(w[f"{p}.q"]).T).view(T, H, D)
    k = silu(h @ d(w[f"{p}.k"]).T).view(T, H, D)
    v = silu(h @ d(w[f"{p}.v"]).T).view(T, H, V)
    decay = [float(x) for x in m["decay"]]
    o = torch.zeros((T, H, V), dtype=F64)
    for a in range(H):
        S = torch.zeros((D, V), dtype=F64)
        for t in range(T):
            S = decay[a] * S + k[t, a][:, None] * v[t, a][None, :]
            o[t, a] = S.T @ q[t, a]
    o = rms_unit(o.reshape(T, H * V), eps) * d(w[f"{p}.norm"])
    return (o * torch.sigmoid(h @ d(w[f"{p}.g"]).T)) @ d(w[f"{p}.o"]).T


def parallel_mixer(h, w, p, m, eps):
    return float(m["left_scale"]) * chunked_attention(h, w, f"{p}.left", m["left"], eps) + \
        float(m["right_scale"]) * decayed_linear_attention(h, w, f"{p}.right", m["right"], eps)


# ------------------------------------------------------------------------------------------ the selective scan
def selective_scan_mixer(h, w, p, m):
    T = h.shape[0]
    inner, N, R, taps = int(m["inner"]), int(m["state"]), int(m["dt_rank"]), int(m["conv"])
    xz = h @ d(w[f"{p}.in"]).T
    x, z = xz[:, :inner], xz[:, inner:]
    cw = d(w[f"{p}.conv"])                                            # [inner, taps], the last column is the current token's
    padded = torch.cat([torch.zeros((taps - 1, inner), dtype=F64), x], 0)
    c = d(w[f"{p}.conv.b"]).expand(T, inner).clone()
    for j in range(taps):
        c = c + cw[:, j] * padded[j:j + T]
    x = silu(c)
    low = x @ d(w[f"{p}.x"]).T
    dt_low, B, C = low[:, :R], low[:, R:R + N], low[:, R + N:R + 2 * N]
    dt = softplus(dt_low @ d(w[f"{p}.dt"]).T + d(w[f"{p}.dt.b"]))    # [T, inner]
    A = -torch.exp(d(w[f"{p}.A_log"]))                                # [inner, N]
    S = torch.zeros((inner, N), dtype=F64)
    y = torch.zeros((T, inner), dtype=F64)
    for t in range(T):
        S = torch.exp(dt[t][:, None] * A) * S + (dt[t] * x[t])[:, None] * B[t][None, :]
        y[t] = S @ C[t] + d(w[f"{p}.D"]) * x[t]
    return (y * silu(z)) @ d(w[f"{p}.o"]).T


# ------------------------------------------------------------------------------------------ the model
def layer_runs(cfg):
    """[(layer, pass number or None when the run is not the first of a pass)] in the order the layers run."""
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop:
        return [(i, None) for i in range(n)]
    start, stop, times = int(loop["start"]), int(loop["stop"]), int(loop["times"])
    runs = [(i, None) for i in range(start)]
    for t in range(times):
        runs += [(i, t if i == start else None) for i in range(start, stop)]
    return runs + [(i, None) for i in range(stop, n)]


def layer(x, cfg, w, i):
    eps, l, p = float(cfg["norm"]["eps"]), cfg["layers"][i], f"l{i}"
    h = token_shift(scalar_norm(x, w[f"{p}.norm1"], eps), w[f"{p}.shift"])
    if l["type"] == "parallel":
        x = x + parallel_mixer(h, w, f"{p}.mix", l["mixer"], eps)
    elif l["type"] == "mamba1":
        x = x + selective_scan_mixer(h, w, f"{p}.mix", l["mixer"])
    else:
        raise ValueError(l["type"])
    if l.get("mlp") is not None:
        x = x + dense_ff(scalar_norm(x, w[f"{p}.norm2"], eps), w, f"{p}.mlp")
    return x


def hidden_states(cfg, w, tokens):
    """The residual stream after every layer run, [runs, T, W]."""
    x0 = d(w["embed"])[torch.as_tensor(tokens, dtype=torch.long)]
    x, out = x0, []
    for i, t in layer_runs(cfg):
        if t is not None:
            x = torch.cat([x, x0], -1) @ d(w["loop.in"]).T + d(w["loop.step"])[t]
        x = layer(x, cfg, w, i)
        out.append(x)
    return torch.stack(out)


def logits(cfg, w, tokens):
    """Logits at every position of one sequence, float64 [T, vocab]."""
    x = hidden_states(cfg, w, tokens)[-1]
    return scalar_norm(x, w["final.norm"], float(cfg["norm"]["eps"])) @ d(w["head"]).T


class PlainLulenex:
    """A model folder (config.json, model.safetensors) read without the engine's loader."""

    def __init__(self, model_dir):
        import json
        import struct
        from pathlib import Path

        import numpy as np
        model_dir = Path(model_dir)
        self.cfg = json.loads((model_dir / "config.json").read_text())
        raw = (model_dir / "model.safetensors").read_bytes()
        n = struct.unpack("<Q", raw[:8])[0]
        header = json.loads(raw[8:8 + n])
        self.w = {}
        for name, info in header.items():
            if name == "__metadata__":
                continue
            a, b = info["data_offsets"]
            data = raw[8 + n + a:8 + n + b]
            if info["dtype"] == "BF16":
                bits = np.frombuffer(data, dtype="<u2").astype(np.uint32) << 16
                t = torch.from_numpy(bits.view(np.float32).copy())
            elif info["dtype"] == "F32":
                t = torch.from_numpy(np.frombuffer(data, dtype="<f4").copy())
            else:
                raise ValueError(f"{name}: dtype {info['dtype']}")
            self.w[name] = t.reshape(info["shape"]).to(F64)

    def logits(self, tokens):
        return logits(self.cfg, self.w, tokens)

    def hidden_states(self, tokens):
        return hidden_states(self.cfg, self.w, tokens)

    def greedy(self, prompt, n):
        toks, out = list(prompt), []
        for _ in range(n):
            out.append(int(self.logits(toks)[-1].argmax()))
            toks.append(out[-1])
        return out
