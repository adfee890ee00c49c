"""Typed configuration of the Ditalorn decoder, read from its own config.json keys.

A Ditalorn model is a list of layers; a layer has a mixer, which is windowed latent attention with a query latent and an output gate or
grouped attention with sigmoid weights behind a short convolution of its projections, and a mixture of experts as its feed-forward (or
none). config.json gives every size and every constant that differs between models; nothing here fixes one.

    architecture     "Ditalorn"
    vocab, width     vocabulary size and width of the residual stream
    max_positions    rows of the table of learned position vectors
    embedding.scale  factor on a token's vector (1 when absent)
    norm.eps         epsilon of every RMS norm
    layers[i]        type "latent_attention": mixer {heads, dim, vdim, kv_rank, q_rank, scale, mask {size}?}
                     type "attention":        mixer {heads, kv_heads?, dim, vdim, scale, conv?, q_temp {coef, every}?}
                     mlp null | {kind "moe", expert {ff}, router {experts, top, groups {count, keep}?}}
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Mapping, Optional

from . import ConfigError

MIXER_TYPES = ("latent_attention", "attention")


def _need(d: Mapping[str, Any], key: str, where: str):
    if not isinstance(d, Mapping) or d.get(key) is None:
        raise ConfigError(f"config.json has no {where}.{key}")
    return d[key]


@dataclass(frozen=True)
class LatentMixerConfig:
    heads: int
    dim: int                  # query/key values per head
    vdim: int                 # value size per head
    kv_rank: int              # size of the cached latent
    q_rank: int               # size of the queries' latent
    scale: float              # factor on the scores
    window: Optional[int]     # a position sees itself and the window - 1 positions before it; None: all

    @classmethod
    def from_dict(cls, m: Mapping[str, Any], where: str) -> "LatentMixerConfig":
        mask = m.get("mask") or {}
        c = cls(heads=int(_need(m, "heads", where)), dim=int(_need(m, "dim", where)), vdim=int(_need(m, "vdim", where)), kv_rank=int(_need(m, "kv_rank", where)),
                q_rank=int(_need(m, "q_rank", where)), scale=float(_need(m, "scale", where)), window=None if mask.get("size") is None else int(mask["size"]))
        for name in ("heads", "dim", "vdim", "kv_rank", "q_rank"):
            if getattr(c, name) <= 0:
                raise ConfigError(f"{where}.{name} must be positive, got {getattr(c, name)}")
        if c.kv_rank > 1024:
            raise ConfigError(f"{where}.kv_rank {c.kv_rank} is above the 1024 the attention kernel holds")
        if c.window is not None and c.window <= 0:
            raise ConfigError(f"{where}.mask.size must be positive, got {c.window}")
        return c

    def to_dict(self) -> dict[str, Any]:
        d: dict[str, Any] = {"heads": self.heads, "dim": self.dim, "vdim": self.vdim, "kv_rank": self.kv_rank, "q_rank": self.q_rank, "scale": self.scale}
        if self.window is not None:
            d["mask"] = {"size": self.window}
        return d


@dataclass(frozen=True)
class SigmoidMixerConfig:
    heads: int
    kv_heads: int
    dim: int                          # query/key size per head
    vdim: int                         # value size per head
    scale: float                      # factor on the scores
    conv: int                         # taps of the convolution on q, k and v (0: none)
    q_temp: Optional[tuple]           # (coef, every) of the query temperature; None: none

    @classmethod
    def from_dict(cls, m: Mapping[str, Any], where: str) -> "SigmoidMixerConfig":
        qt = m.get("q_temp")
        c = cls(heads=int(_need(m, "heads", where)), kv_heads=int(m.get("kv_heads") or m["heads"]), dim=int(_need(m, "dim", where)), vdim=int(m.get("vdim") or m["dim"]),
                scale=float(_need(m, "scale", where)), conv=int(m.get("conv") or 0),
                q_temp=None if not qt else (float(_need(qt, "coef", where + ".q_temp")), int(_need(qt, "every", where + ".q_temp"))))
        if c.heads <= 0 or c.kv_heads <= 0 or c.heads % c.kv_heads:
            raise ConfigError(f"{where}: {c.heads} heads are not a positive multiple of {c.kv_heads} kv_heads")
        if c.dim <= 0 or c.vdim <= 0 or max(c.dim, c.vdim) > 256:
            raise ConfigError(f"{where}: dim {c.dim} and vdim {c.vdim} must be positive and at most 256")
        if c.conv < 0:
            raise ConfigError(f"{where}.conv must not be negative, got {c.conv}")
        if c.q_temp is not None and c.q_temp[1] <= 0:
            raise ConfigError(f"{where}.q_temp.every must be positive, got {c.q_temp[1]}")
        return c

    def to_dict(self) -> dict[str, Any]:
        d: dict[str, Any] = {"heads": self.heads, "kv_heads": self.kv_heads, "dim": self.dim, "vdim": self.vdim, "scale": self.scale}
        if self.conv:
            d["conv"] = self.conv
        if self.q_temp is not None:
            d["q_temp"] = {"coef": self.q_temp[0], "every": self.q_temp[1]}
        return d


@dataclass(frozen=True)
class ExpertsConfig:
    ff: int             # one expert's inner size
    experts: int
    top: int            # experts a token uses
    groups: int         # experts lie in this many equal groups of neighbours
    groups_keep: int    # only experts of the best groups_keep groups can be chosen

    @classmethod
    def from_dict(cls, f: Mapping[str, Any], where: str) -> "ExpertsConfig":
        kind = _need(f, "kind", where)
        if kind != "moe":
            raise ConfigError(f"{where}.kind {kind!r} is not supported (known: moe)")
        r = _need(f, "router", where)
        g = r.get("groups") or {}
        c = cls(ff=int(_need(_need(f, "expert", where), "ff", where + ".expert")), experts=int(_need(r, "experts", where + ".router")),
                top=int(_need(r, "top", where + ".router")), groups=int(g.get("count") or 1), groups_keep=int(g.get("keep") or g.get("count") or 1))
        if c.ff <= 0 or c.experts <= 0 or not 0 < c.top <= c.experts:
            raise ConfigError(f"{where}: inner size {c.ff}, top {c.top} of {c.experts} experts")
        if c.groups <= 0 or c.experts % c.groups or not 0 < c.groups_keep <= c.groups:
            raise ConfigError(f"{where}.router.groups: {c.experts} experts do not form {c.groups} equal groups of which {c.groups_keep} stay")
        if c.top > c.groups_keep * (c.experts // c.groups):
            raise ConfigError(f"{where}.router: {c.top} experts a token cannot come from {c.groups_keep} groups of {c.experts // c.groups}")
        return c

    def to_dict(self) -> dict[str, Any]:
        return {"kind": "moe", "expert": {"ff": self.ff}, "router": {"experts": self.experts, "top": self.top, "groups": {"count": self.groups, "keep": self.groups_keep}}}


@dataclass(frozen=True)
class DitalornLayer:
    type: str
    mixer: Any                          # LatentMixerConfig | SigmoidMixerConfig
    mlp: Optional[ExpertsConfig]


@dataclass(frozen=True)
class DitalornConfig:
    vocab: int
    width: int
    max_positions: int
    embedding_scale: float
    norm_eps: float
    layers: tuple[DitalornLayer, ...]
    architecture: str = "Ditalorn"

    @property
    def num_layers(self) -> int:
        return len(self.layers)

    @classmethod
    def from_dict(cls, raw: Mapping[str, Any]) -> "DitalornConfig":
        layers_raw = _need(raw, "layers", "config")
        if not isinstance(layers_raw, (list, tuple)) or not layers_raw:
            raise ConfigError("config.json: layers must be a non-empty list")
        layers = []
        for i, l in enumerate(layers_raw):
            t, where = _need(l, "type", f"layers[{i}]"), f"layers[{i}].mixer"
            if t == "latent_attention":
                mixer = LatentMixerConfig.from_dict(_need(l, "mixer", f"layers[{i}]"), where)
            elif t == "attention":
                mixer = SigmoidMixerConfig.from_dict(_need(l, "mixer", f"layers[{i}]"), where)
            else:
                raise ConfigError(f"layers[{i}].type {t!r} is not supported (known: {', '.join(MIXER_TYPES)})")
            layers.append(DitalornLayer(t, mixer, None if l.get("mlp") is None else ExpertsConfig.from_dict(l["mlp"], f"layers[{i}].mlp")))
        cfg = cls(vocab=int(_need(raw, "vocab", "config")), width=int(_need(raw, "width", "config")), max_positions=int(_need(raw, "max_positions", "config")),
                  embedding_scale=float((raw.get("embedding") or {}).get("scale", 1.0)), norm_eps=float(_need(_need(raw, "norm", "config"), "eps", "norm")),
                  layers=tuple(layers), architecture=str(raw.get("architecture", "Ditalorn")))
        if cfg.vocab <= 0 or cfg.width <= 0 or cfg.max_positions <= 0 or not cfg.norm_eps > 0:
            raise ConfigError(f"vocab {cfg.vocab}, width {cfg.width}, max_positions {cfg.max_positions} and norm.eps {cfg.norm_eps} must be positive")
        return cfg

    def to_dict(self) -> dict[str, Any]:
        return {"architecture": self.architecture, "vocab": self.vocab, "width": self.width, "max_positions": self.max_positions,
                "embedding": {"scale": self.embedding_scale}, "norm": {"eps": self.norm_eps},
                "layers": [{"type": l.type, "mixer": l.mixer.to_dict(), "mlp": None if l.mlp is None else l.mlp.to_dict()} for l in self.layers]}
