"""Tiny Ditalorn configurations for the tests, with weights the tests make themselves. They differ in every size and constant: width (a
multiple of 8 or not), the order of the two kinds of layer, head counts (equal, grouped by two, four and sixteen), key and value sizes
(equal or not, multiples of 16 or not), latents of the queries and of the keys (multiples of 16 or not), windows of one position, shorter
and longer than the prompts and absent, the convolution's length (none; one tap: no state; two to four), a query temperature whose period
passes inside the prompts or none, experts a token (one to four) in one to four groups of which one to all stay, layers without a
feed-forward, embedding scale, norm epsilon, page size."""
from __future__ import annotations

import json
from pathlib import Path

import torch


def _lat(heads, dim, vdim, kv_rank, q_rank, scale, window):
    m = {"heads": heads, "dim": dim, "vdim": vdim, "kv_rank": kv_rank, "q_rank": q_rank, "scale": scale}
    if window is not None:
        m["mask"] = {"size": window}
    return m


def _att(heads, kv_heads, dim, vdim, scale, conv, q_temp):
    m = {"heads": heads, "dim": dim, "vdim": vdim, "scale": scale}
    if kv_heads is not None:
        m["kv_heads"] = kv_heads
    if conv:
        m["conv"] = conv
    if q_temp:
        m["q_temp"] = {"coef": q_temp[0], "every": q_temp[1]}
    return m


def _moe(ff, experts, top, groups=None):
    r = {"experts": experts, "top": top}
    if groups:
        r["groups"] = {"count": groups[0], "keep": groups[1]}
    return {"kind": "moe", "expert": {"ff": ff}, "router": r}


def _layer(kind, mixer, mlp):
    return {"type": kind, "mixer": mixer, "mlp": mlp}


CONFIGS = {
    # sigmoid attention first; two key/value heads of unequal key and value size, four taps, a temperature that changes every 16 positions; latents
    # that are multiples of 16 with a window shorter than the prompts, and one longer than every prompt; layers without a feed-forward after
    # either kind of mixer; three groups of which two stay
    "A": dict(seed=31, page_size=16, config={
        "architecture": "Ditalorn", "vocab": 300, "width": 80, "max_positions": 256, "embedding": {"scale": 3.0}, "norm": {"eps": 1e-5},
        "layers": [_layer("attention", _att(4, 2, 32, 16, 0.2, 4, (0.7, 16)), _moe(24, 6, 2, (3, 2))),
                   _layer("latent_attention", _lat(3, 16, 24, 32, 48, 0.25, 9), _moe(40, 4, 2)),
                   _layer("latent_attention", _lat(2, 32, 16, 16, 16, 0.2, 1000), None),
                   _layer("attention", _att(2, 1, 16, 48, 0.3, 2, (0.3, 5)), None)]}),
    # a width that is no multiple of 8 (the plain product also in bfloat16); no embedding scale; sizes that are no multiples of 16 (the plain attention
    # kernels also in bfloat16); as many key/value heads as heads (the key left out); one tap (no state) and no convolution at all; no temperature;
    # a window of one position and no window; one expert a token; groups that all stay; small pages
    "B": dict(seed=32, page_size=8, config={
        "architecture": "Ditalorn", "vocab": 257, "width": 132, "max_positions": 200, "norm": {"eps": 1e-6},
        "layers": [_layer("latent_attention", _lat(5, 24, 40, 24, 20, 0.2, 1), _moe(36, 7, 1)),
                   _layer("attention", _att(5, None, 24, 40, 0.2, 1, None), _moe(20, 4, 1, (2, 2))),
                   _layer("latent_attention", _lat(2, 8, 8, 40, 72, 0.35, None), _moe(36, 6, 3, (2, 1))),
                   _layer("attention", _att(3, 1, 40, 24, 0.15, 0, (1.5, 3)), _moe(36, 7, 1))]}),
    # the sizes the tensor-core kernels take: groups of four and of sixteen query heads, heads of 32 to 128, latents of 128 and 64, experts whose inner
    # size is a multiple of 64, four experts a token from two of four groups, larger pages
    "C": dict(seed=33, page_size=32, config={
        "architecture": "Ditalorn", "vocab": 512, "width": 256, "max_positions": 512, "embedding": {"scale": 16.0}, "norm": {"eps": 1e-5},
        "layers": [_layer("latent_attention", _lat(8, 64, 64, 128, 96, 0.125, 48), _moe(64, 16, 4, (4, 2))),
                   _layer("attention", _att(8, 2, 64, 128, 0.125, 3, (0.5, 64)), _moe(64, 8, 2, (2, 1))),
                   _layer("attention", _att(16, 1, 32, 32, 0.18, 2, (0.25, 7)), _moe(128, 4, 1)),
                   _layer("latent_attention", _lat(4, 128, 32, 64, 64, 0.09, 17), _moe(64, 16, 4, (4, 2)))]}),
}


def tensors(config: dict, seed: int) -> dict[str, torch.Tensor]:
    """Random bfloat16 tensors: matrices N(0, gain / sqrt(fan-in)) so that activations stay of order one, norm weights around zero (the scale is
    1 + w) or around one (the latents' plain norms), taps N(0, 0.5), biases N(0, 0.3), distance-bias numbers in (0.1, 1), a score bias that
    makes the unnormalised weights small, corrections N(0, 0.4) so that choice scores are of both signs."""
    g = torch.Generator().manual_seed(seed)
    W, out = config["width"], {}

    def mat(name, n, k, gain=1.0):
        out[name] = (torch.randn((n, k), generator=g) * gain / k ** 0.5).to(torch.bfloat16)

    def vec(name, n, centre, spread=0.3):
        out[name] = (centre + (torch.rand((n,), generator=g) * 2 - 1) * spread).to(torch.bfloat16)

    def noise(name, shape, std):
        out[name] = (torch.randn(shape, generator=g) * std).to(torch.bfloat16)

    out["embed"] = (torch.randn((config["vocab"], W), generator=g) * 0.3).to(torch.bfloat16)
    noise("pos", (config["max_positions"], W), 0.5)
    for i, l in enumerate(config["layers"]):
        m, p = l["mixer"], f"l{i}"
        H = m["heads"]
        vec(f"{p}.norm1", W, 0.0), vec(f"{p}.norm1b", W, 0.0)
        if l["type"] == "latent_attention":
            mat(f"{p}.mix.dq", m["q_rank"], W), vec(f"{p}.mix.dq.norm", m["q_rank"], 1.0), mat(f"{p}.mix.uq", H * m["dim"], m["q_rank"], 2.0)
            mat(f"{p}.mix.dkv", m["kv_rank"], W), vec(f"{p}.mix.dkv.norm", m["kv_rank"], 1.0)
            mat(f"{p}.mix.uk", H * m["dim"], m["kv_rank"], 2.0), mat(f"{p}.mix.uv", H * m["vdim"], m["kv_rank"])
            mat(f"{p}.mix.g", H, W, 2.0), mat(f"{p}.mix.o", W, H * m["vdim"])
        else:
            G, taps = m.get("kv_heads") or H, m.get("conv") or 0
            sizes = {"q": H * m["dim"], "k": G * m["dim"], "v": G * m["vdim"]}
            for n, rows in sizes.items():
                mat(f"{p}.mix.{n}", rows, W, 2.0 if n != "v" else 1.0), noise(f"{p}.mix.{n}.b", (rows,), 0.3)
                if taps:
                    noise(f"{p}.mix.{n}.conv", (rows, taps), 0.5)
            mat(f"{p}.mix.o", W, H * m["vdim"]), noise(f"{p}.mix.o.b", (W,), 0.3)
            out[f"{p}.mix.r1"] = (0.1 + 0.9 * torch.rand((H,), generator=g)).to(torch.bfloat16)
            out[f"{p}.mix.r2"] = (0.1 + 0.9 * torch.rand((H,), generator=g)).to(torch.bfloat16)
            out[f"{p}.mix.pb"] = (-1.0 + torch.randn((H,), generator=g)).to(torch.bfloat16)
        f = l.get("mlp")
        if f is None:
            continue
        vec(f"{p}.norm2", W, 0.0), vec(f"{p}.norm2b", W, 0.0)
        E = f["router"]["experts"]
        mat(f"{p}.mlp.router", E, W, 2.0), noise(f"{p}.mlp.correction", (E,), 0.4)
        for k in range(E):
            mat(f"{p}.mlp.e{k}.gate", f["expert"]["ff"], W, 2.0), mat(f"{p}.mlp.e{k}.up", f["expert"]["ff"], W, 2.0), mat(f"{p}.mlp.e{k}.down", W, f["expert"]["ff"])
    vec("final.norm", W, 0.0)
    return out


def write_model(name: str, out_dir, config=None, weights=None) -> Path:
    from inference_bench_b200.weights.safetensors_io import write_safetensors
    c = CONFIGS[name]
    out = Path(out_dir)
    out.mkdir(parents=True, exist_ok=True)
    config = config or c["config"]
    (out / "config.json").write_text(json.dumps(config, indent=1))
    write_safetensors(out / "model.safetensors", weights if weights is not None else tensors(config, c["seed"]), {"format": "pt"})
    return out
