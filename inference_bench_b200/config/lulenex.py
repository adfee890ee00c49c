"""Typed configuration of the Lulenex decoder, read from its own config.json keys.

A Lulenex model is a list of layers, some of which may run several times in a row. A layer has a mixer, which is either a selective
scan or two mixers side by side (chunked attention with a sink and a linear recurrence with a fixed decay), and a dense feed-forward
(or none). config.json gives every size and every constant that differs between models; nothing here fixes one.

    architecture   "Lulenex"
    vocab, width   vocabulary size and width of the residual stream
    norm.eps       epsilon of every norm
    loop           null | {start, stop, times}: layers start .. stop - 1 run `times` times in a row
    layers[i]      type "mamba1":   mixer {inner, state, dt_rank, conv}
                   type "parallel": mixer {left {heads, kv_heads, dim, vdim, scale, mask {size}, rot {base, dims}}, left_scale,
                                           right {heads, dim, vdim, decay [heads]}, right_scale}
                   mlp null | {kind "dense", ff}
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Mapping, Optional

from . import ConfigError

MIXER_TYPES = ("mamba1", "parallel")


def _need(d: Mapping[str, Any], key: str, where: str):
    if not isinstance(d, Mapping) or d.get(key) is None:
        raise ConfigError(f"config.json has no {where}.{key}")
    return d[key]


@dataclass(frozen=True)
class ScanMixerConfig:
    inner: int
    state: int
    dt_rank: int
    conv: int       # taps of the causal convolution

    @classmethod
    def from_dict(cls, m: Mapping[str, Any], where: str) -> "ScanMixerConfig":
        c = cls(*(int(_need(m, k, where)) for k in ("inner", "state", "dt_rank", "conv")))
        if min(c.inner, c.state, c.dt_rank, c.conv) <= 0 or c.state > 256:
            raise ConfigError(f"{where}: inner {c.inner}, state {c.state} (at most 256), dt_rank {c.dt_rank} and conv {c.conv} must be positive")
        return c

    def to_dict(self) -> dict[str, Any]:
        return {"inner": self.inner, "state": self.state, "dt_rank": self.dt_rank, "conv": self.conv}


@dataclass(frozen=True)
class ChunkAttentionConfig:
    heads: int
    kv_heads: int
    dim: int            # query/key size per head; the values are the keys, so it is the value size too
    scale: float
    chunk: int          # a position sees the earlier positions of its own block of this many
    rot_base: float
    rot_dims: int

    @classmethod
    def from_dict(cls, m: Mapping[str, Any], where: str) -> "ChunkAttentionConfig":
        rot = _need(m, "rot", where)
        c = cls(heads=int(_need(m, "heads", where)), kv_heads=int(m.get("kv_heads") or m["heads"]), dim=int(_need(m, "dim", where)),
                scale=float(_need(m, "scale", where)), chunk=int(_need(_need(m, "mask", where), "size", where + ".mask")),
                rot_base=float(_need(rot, "base", where + ".rot")), rot_dims=int(_need(rot, "dims", where + ".rot")))
        if m.get("vdim") is not None and int(m["vdim"]) != c.dim:
            raise ConfigError(f"{where}: the values are the keys, so vdim {m['vdim']} must equal dim {c.dim}")
        if c.heads <= 0 or c.kv_heads <= 0 or c.heads % c.kv_heads:
            raise ConfigError(f"{where}: {c.heads} heads are not a positive multiple of {c.kv_heads} kv_heads")
        if c.dim <= 0 or c.dim % 2 or c.dim > 256:
            raise ConfigError(f"{where}: dim {c.dim} must be even, positive and at most 256")
        if c.rot_dims < 0 or c.rot_dims % 2 or c.rot_dims > c.dim or not c.rot_base > 0:
            raise ConfigError(f"{where}.rot: dims {c.rot_dims} must be even and at most dim {c.dim}, base {c.rot_base} positive")
        if c.chunk <= 0:
            raise ConfigError(f"{where}.mask.size must be positive, got {c.chunk}")
        return c

    def to_dict(self) -> dict[str, Any]:
        return {"heads": self.heads, "kv_heads": self.kv_heads, "dim": self.dim, "vdim": self.dim, "scale": self.scale, "mask": {"size": self.chunk},
                "rot": {"base": self.rot_base, "dims": self.rot_dims}}


@dataclass(frozen=True)
class DecayedLinearConfig:
    heads: int
    dim: int
    vdim: int
    decay: tuple

    @classmethod
    def from_dict(cls, m: Mapping[str, Any], where: str) -> "DecayedLinearConfig":
        decay = _need(m, "decay", where)
        c = cls(heads=int(_need(m, "heads", where)), dim=int(_need(m, "dim", where)), vdim=int(_need(m, "vdim", where)),
                decay=tuple(float(d) for d in (decay if isinstance(decay, (list, tuple)) else [decay] * int(m["heads"]))))
        if c.heads <= 0 or c.dim <= 0 or c.vdim <= 0 or c.dim > 512:
            raise ConfigError(f"{where}: heads {c.heads}, dim {c.dim} (at most 512) and vdim {c.vdim} must be positive")
        if len(c.decay) != c.heads or any(not 0.0 <= d <= 1.0 for d in c.decay):
            raise ConfigError(f"{where}.decay must give {c.heads} numbers in [0, 1], got {list(c.decay)}")
        return c

    def to_dict(self) -> dict[str, Any]:
        return {"heads": self.heads, "dim": self.dim, "vdim": self.vdim, "decay": list(self.decay)}


@dataclass(frozen=True)
class ParallelMixerConfig:
    left: ChunkAttentionConfig
    right: DecayedLinearConfig
    left_scale: float
    right_scale: float

    @classmethod
    def from_dict(cls, m: Mapping[str, Any], where: str) -> "ParallelMixerConfig":
        return cls(ChunkAttentionConfig.from_dict(_need(m, "left", where), where + ".left"), DecayedLinearConfig.from_dict(_need(m, "right", where), where + ".right"),
                   float(_need(m, "left_scale", where)), float(_need(m, "right_scale", where)))

    def to_dict(self) -> dict[str, Any]:
        return {"left": self.left.to_dict(), "left_scale": self.left_scale, "right": self.right.to_dict(), "right_scale": self.right_scale}


@dataclass(frozen=True)
class LulenexLayer:
    type: str
    mixer: Any              # ScanMixerConfig | ParallelMixerConfig
    ff: Optional[int]       # inner size of the dense feed-forward, None for a layer without one


@dataclass(frozen=True)
class Loop:
    start: int
    stop: int
    times: int


@dataclass(frozen=True)
class LulenexConfig:
    vocab: int
    width: int
    norm_eps: float
    layers: tuple
    loop: Optional[Loop]
    architecture: str = "Lulenex"

    @property
    def num_layers(self) -> int:
        return len(self.layers)

    def runs(self) -> list:
        """[(layer, pass number when the run opens a pass, else None)] in the order the layers run."""
        n, lp = len(self.layers), self.loop
        if lp is None:
            return [(i, None) for i in range(n)]
        out = [(i, None) for i in range(lp.start)]
        for t in range(lp.times):
            out += [(i, t if i == lp.start else None) for i in range(lp.start, lp.stop)]
        return out + [(i, None) for i in range(lp.stop, n)]

    @classmethod
    def from_dict(cls, raw: Mapping[str, Any]) -> "LulenexConfig":
        layers_raw = _need(raw, "layers", "config")
        if not isinstance(layers_raw, (list, tuple)) or not layers_raw:
            raise ConfigError("config.json: layers must be a non-empty list")
        layers = []
        for i, l in enumerate(layers_raw):
            t, where = _need(l, "type", f"layers[{i}]"), f"layers[{i}].mixer"
            if t == "mamba1":
                mixer = ScanMixerConfig.from_dict(_need(l, "mixer", f"layers[{i}]"), where)
            elif t == "parallel":
                mixer = ParallelMixerConfig.from_dict(_need(l, "mixer", f"layers[{i}]"), where)
            else:
                raise ConfigError(f"layers[{i}].type {t!r} is not supported (known: {', '.join(MIXER_TYPES)})")
            mlp, ff = l.get("mlp"), None
            if mlp is not None:
                if _need(mlp, "kind", f"layers[{i}].mlp") != "dense":
                    raise ConfigError(f"layers[{i}].mlp.kind {mlp['kind']!r} is not supported (known: dense)")
                ff = int(_need(mlp, "ff", f"layers[{i}].mlp"))
                if ff <= 0:
                    raise ConfigError(f"layers[{i}].mlp.ff must be positive, got {ff}")
            layers.append(LulenexLayer(t, mixer, ff))
        loop = None
        if raw.get("loop") is not None:
            lr = raw["loop"]
            loop = Loop(int(_need(lr, "start", "loop")), int(_need(lr, "stop", "loop")), int(_need(lr, "times", "loop")))
            if not 0 <= loop.start < loop.stop <= len(layers) or loop.times < 1:
                raise ConfigError(f"loop: layers {loop.start} .. {loop.stop - 1} of {len(layers)}, {loop.times} times, is not a loop")
        cfg = cls(vocab=int(_need(raw, "vocab", "config")), width=int(_need(raw, "width", "config")),
                  norm_eps=float(_need(_need(raw, "norm", "config"), "eps", "norm")), layers=tuple(layers), loop=loop,
                  architecture=str(raw.get("architecture", "Lulenex")))
        if cfg.vocab <= 0 or cfg.width <= 0 or not cfg.norm_eps > 0:
            raise ConfigError(f"vocab {cfg.vocab}, width {cfg.width} and norm.eps {cfg.norm_eps} must be positive")
        return cfg

    def to_dict(self) -> dict[str, Any]:
        return {"architecture": self.architecture, "vocab": self.vocab, "width": self.width, "norm": {"eps": self.norm_eps},
                "loop": None if self.loop is None else {"start": self.loop.start, "stop": self.loop.stop, "times": self.loop.times},
                "layers": [{"type": l.type, "mixer": l.mixer.to_dict(), "mlp": None if l.ff is None else {"kind": "dense", "ff": l.ff}} for l in self.layers]}
