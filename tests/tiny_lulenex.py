"""Tiny Lulenex configurations for the tests, with weights the tests make themselves. They differ in every size and constant: width (a
multiple of 8 or not), the order of scan and parallel layers, a loop at the start, in the middle up to the last layer, of one pass, or
none; query and key/value head counts (equal, grouped by two, by eight), head sizes with part, all or none of a head turned, blocks of
positions shorter than a page, equal to one, and longer than every prompt; decays of 0 and 1 among the heads; one to four taps (one tap:
no convolution state); 3 to 40 states a channel, step ranks of 1 to 8; layers without a feed-forward after either mixer; norm epsilon,
page size."""
from __future__ import annotations

import json
from pathlib import Path

import torch


def _par(heads, kv_heads, dim, chunk, dims, base, scale, rheads, rdim, rvdim, decay, left_scale, right_scale):
    return {"left": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim, "mask": {"size": chunk}, "rot": {"base": base, "dims": dims}, "scale": scale},
            "left_scale": left_scale, "right": {"heads": rheads, "dim": rdim, "vdim": rvdim, "decay": list(decay)}, "right_scale": right_scale}


def _scan(inner, state, dt_rank, conv):
    return {"inner": inner, "state": state, "dt_rank": dt_rank, "conv": conv}


def _layer(kind, mixer, ff):
    return {"type": kind, "mixer": mixer, "mlp": None if ff is None else {"kind": "dense", "ff": ff}}


CONFIGS = {
    # a scan first; a loop over the first two layers, three passes; grouped attention with half of a head turned and blocks of 7 positions
    # (shorter than a page); layers without a feed-forward after a parallel mixer and after a scan
    "A": dict(seed=31, page_size=16, config={
        "architecture": "Lulenex", "vocab": 300, "width": 80, "norm": {"eps": 1e-5}, "loop": {"start": 0, "stop": 2, "times": 3},
        "layers": [_layer("mamba1", _scan(96, 5, 3, 4), 40),
                   _layer("parallel", _par(4, 2, 32, 7, 16, 1000.0, 0.3, 3, 16, 24, (0.5, 0.9, 0.99), 1.3, 0.4), 56),
                   _layer("parallel", _par(2, 2, 16, 20, 16, 50.0, 0.5, 2, 40, 8, (0.97, 0.2), 0.6, 1.1), None),
                   _layer("mamba1", _scan(48, 12, 8, 2), None)]}),
    # a width that is no multiple of 8; no loop; as many kv heads as query heads; nothing of a head turned; blocks longer than every prompt;
    # decays of 1 and 0; one tap (no convolution state); a step rank of 1
    "B": dict(seed=32, page_size=8, config={
        "architecture": "Lulenex", "vocab": 257, "width": 132, "norm": {"eps": 1e-6}, "loop": None,
        "layers": [_layer("parallel", _par(6, 6, 24, 1000, 0, 10.0, 0.25, 4, 12, 20, (1.0, 0.0, 0.8, 0.999), 1.0, 1.0), 36),
                   _layer("mamba1", _scan(60, 17, 1, 1), 100),
                   _layer("parallel", _par(3, 1, 10, 13, 10, 300.0, 0.7, 1, 48, 20, (0.95,), 0.3, 2.0), 36)]}),
    # heads of 64 and 128, eight query heads on one kv head, blocks as long as a page and of three pages, a loop from the second layer to the
    # last, a scan inside the loop, three taps
    "C": dict(seed=33, page_size=16, config={
        "architecture": "Lulenex", "vocab": 512, "width": 256, "norm": {"eps": 1e-5}, "loop": {"start": 1, "stop": 3, "times": 2},
        "layers": [_layer("parallel", _par(8, 1, 64, 16, 64, 10000.0, 0.125, 4, 64, 64, (0.9, 0.99, 0.999, 0.7), 0.8, 0.5), 64),
                   _layer("mamba1", _scan(128, 40, 4, 3), 128),
                   _layer("parallel", _par(2, 2, 128, 48, 32, 500000.0, 0.09, 2, 32, 128, (0.98, 0.6), 1.0, 0.25), 96)]}),
    # one layer, looped once
    "D": dict(seed=34, page_size=32, config={
        "architecture": "Lulenex", "vocab": 100, "width": 48, "norm": {"eps": 1e-6}, "loop": {"start": 0, "stop": 1, "times": 1},
        "layers": [_layer("parallel", _par(2, 1, 12, 5, 4, 100.0, 0.4, 2, 8, 8, (0.9, 0.5), 1.0, 1.0), 24)]}),
}


def tensors(config: dict, seed: int) -> dict[str, torch.Tensor]:
    """Random bfloat16 tensors: matrices N(0, gain / sqrt(fan-in)) so that activations stay of order one, norm numbers around one, shift
    weights in (0, 1), sinks N(0, 1), decay rates between 0.5 and 8, step biases around -1, biases N(0, 0.3)."""
    g = torch.Generator().manual_seed(seed)
    W, out = config["width"], {}

    def mat(name, n, k, gain=1.0):
        out[name] = (torch.randn((n, k), generator=g) * gain / k ** 0.5).to(torch.bfloat16)

    def noise(name, shape, std, centre=0.0):
        out[name] = (centre + torch.randn(shape, generator=g) * std).to(torch.bfloat16)

    def number(name):
        out[name] = (0.7 + 0.6 * torch.rand((), generator=g)).to(torch.bfloat16)

    out["embed"] = torch.randn((config["vocab"], W), generator=g).to(torch.bfloat16)
    if config.get("loop"):
        mat("loop.in", W, 2 * W, 1.4), noise("loop.step", (config["loop"]["times"], W), 0.3)
    for i, l in enumerate(config["layers"]):
        m, p = l["mixer"], f"l{i}"
        number(f"{p}.norm1")
        out[f"{p}.shift"] = torch.rand((W,), generator=g).to(torch.bfloat16)
        if l["type"] == "mamba1":
            I, N, R, K = m["inner"], m["state"], m["dt_rank"], m["conv"]
            mat(f"{p}.mix.in", 2 * I, W, 1.5), noise(f"{p}.mix.conv", (I, K), 0.5), noise(f"{p}.mix.conv.b", (I,), 0.2)
            mat(f"{p}.mix.x", R + 2 * N, I, 1.5), mat(f"{p}.mix.dt", I, R), noise(f"{p}.mix.dt.b", (I,), 1.0, -1.0)
            out[f"{p}.mix.A_log"] = torch.log(0.5 + 7.5 * torch.rand((I, N), generator=g)).to(torch.bfloat16)
            noise(f"{p}.mix.D", (I,), 0.3, 1.0), mat(f"{p}.mix.o", W, I)
        else:
            a, r = m["left"], m["right"]
            H, G, D = a["heads"], a["kv_heads"], a["dim"]
            mat(f"{p}.mix.left.q", H * D, W, 3.0), mat(f"{p}.mix.left.k", G * D, W, 3.0), mat(f"{p}.mix.left.g", H, W, 2.0), mat(f"{p}.mix.left.o", W, H * D)
            noise(f"{p}.mix.left.q.b", (H * D,), 0.3), noise(f"{p}.mix.left.k.b", (G * D,), 0.3), noise(f"{p}.mix.left.o.b", (W,), 0.3), noise(f"{p}.mix.left.sink", (H,), 1.0)
            Hr, Dr, Vr = r["heads"], r["dim"], r["vdim"]
            mat(f"{p}.mix.right.q", Hr * Dr, W), mat(f"{p}.mix.right.k", Hr * Dr, W), mat(f"{p}.mix.right.v", Hr * Vr, W), mat(f"{p}.mix.right.g", Hr * Vr, W, 2.0)
            noise(f"{p}.mix.right.norm", (Hr * Vr,), 0.2, 1.0), mat(f"{p}.mix.right.o", W, Hr * Vr)
        if l.get("mlp") is not None:
            number(f"{p}.norm2")
            mat(f"{p}.mlp.up", l["mlp"]["ff"], W, 1.5), mat(f"{p}.mlp.down", W, l["mlp"]["ff"]), noise(f"{p}.mlp.act", (2,), 0.7)
    number("final.norm")
    mat("head", config["vocab"], W)
    return out


def write_model(name: str, out_dir) -> Path:
    from inference_bench_b200.weights.safetensors_io import write_safetensors
    c = CONFIGS[name]
    out = Path(out_dir)
    out.mkdir(parents=True, exist_ok=True)
    (out / "config.json").write_text(json.dumps(c["config"], indent=1))
    write_safetensors(out / "model.safetensors", tensors(c["config"], c["seed"]), {"format": "pt"})
    return out
