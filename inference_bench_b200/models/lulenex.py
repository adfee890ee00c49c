"""Lulenex as a plan: pre-norm layers with RMS norms whose weight is one number, a token shift in front of every mixer, mixers that are a
selective scan or chunked attention with a sink beside a linear recurrence with a fixed decay, dense feed-forwards with the xIELU
activation, and a run of layers that is repeated with the same weights, each pass entered through a matrix on [stream ; embedding].

Tensor names: `embed`, `loop.in`, `loop.step`, `l<i>.{norm1,norm2,shift}`, `l<i>.mix.{in,conv,conv.b,x,dt,dt.b,A_log,D,o}` or
`l<i>.mix.left.{q,q.b,k,k.b,sink,g,o,o.b}` with `l<i>.mix.right.{q,k,v,g,norm,o}`, `l<i>.mlp.{up,down,act}`, `final.norm`, `head`.
They have no common root. A layer that runs in several passes has one schedule entry per pass, so every pass has its own cache and state.
"""
from __future__ import annotations

from ..config.lulenex import LulenexConfig
from ..parts.plan import LayerPlan, ModelPlan, PartSpec, ScheduleEntry
from ..registry import register_architecture

MAX_POSITIONS = 1 << 20   # the rotation has no table: positions are bounded by the cache alone


def lulenex_plan(c: LulenexConfig) -> ModelPlan:
    layers = []
    norm = lambda name: PartSpec("rmsnorm", {"name": name, "size": c.width, "eps": c.norm_eps, "scalar": True})
    for i, l in enumerate(c.layers):
        m, p = l.mixer, f"l{i}"
        if l.type == "mamba1":
            mixer = PartSpec("mamba1", {"prefix": f"{p}.mix", "hidden": c.width, "inner": m.inner, "state": m.state, "dt_rank": m.dt_rank, "taps": m.conv})
        else:
            a, r = m.left, m.right
            rope = PartSpec("rope", {"rotary_dim": a.rot_dims, "theta": a.rot_base}) if a.rot_dims else PartSpec("none")
            mixer = PartSpec("parallel", {"hidden": c.width, "branches": (
                ("chunk_attention", m.left_scale, {"prefix": f"{p}.mix.left", "heads": a.heads, "kv_heads": a.kv_heads, "head_dim": a.dim, "chunk": a.chunk,
                                                   "scale": a.scale, "norm_eps": c.norm_eps, "position": rope}),
                ("decayed_linear", m.right_scale, {"prefix": f"{p}.mix.right", "heads": r.heads, "dim": r.dim, "vdim": r.vdim, "decay": r.decay,
                                                   "norm_eps": c.norm_eps}))})
        if l.ff is None:
            ff, ff_norm = PartSpec("none"), PartSpec("none")
        else:
            ff, ff_norm = PartSpec("dense_xielu", {"prefix": f"{p}.mlp", "hidden": c.width, "intermediate": l.ff}), norm(f"{p}.norm2")
        layers.append(LayerPlan(prefix=p, block="prenorm_shift", mixer=mixer, feed_forward=ff, mixer_norm=norm(f"{p}.norm1"), feed_forward_norm=ff_norm,
                                block_params=(("prefix", p), ("hidden", c.width))))
    return ModelPlan(
        architecture="Lulenex", vocab_size=c.vocab, hidden_size=c.width, max_positions=MAX_POSITIONS,
        embedding=PartSpec("table", {"name": "embed", "vocab": c.vocab, "hidden": c.width}),
        layers=tuple(layers), schedule=tuple(ScheduleEntry(i, enter=None if t is None else (0, t)) for i, t in c.runs()),
        stream_parts=() if c.loop is None else (PartSpec("loop_entry", {"hidden": c.width, "passes": c.loop.times}),),
        final_norm=norm("final.norm"), head=PartSpec("linear", {"name": "head", "vocab": c.vocab, "hidden": c.width}),
        ignored_tensors=tuple(f"l{i}.norm2" for i, l in enumerate(c.layers) if l.ff is None),
        root="",
    )


register_architecture(["Lulenex", "lulenex"], LulenexConfig.from_dict, lulenex_plan,
                      traits={"attention": "gqa", "qk_norm": True, "norm": "rmsnorm", "norm_unit_offset": False, "rope_style": "neox", "activation": "xielu"})
