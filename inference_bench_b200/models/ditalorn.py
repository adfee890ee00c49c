"""Ditalorn as a plan: layers with an RMS norm (weight stored around zero) in front of every sublayer and another on what it gives back;
mixers are windowed latent attention (queries through a latent of their own, no rotated part, a sigmoid gate per head on the output) or
grouped attention with sigmoid weights (biased projections behind a short causal convolution, a query temperature, unit-normed values, a
distance bias and a bias per head on the scores); feed-forwards are experts chosen by sigmoid scores plus a correction, within the best
groups by the sum of their two largest choice scores, weighted by the plain scores. The embedding multiplies the token's vector by a
constant and adds a learned vector per position; the head is the embedding table itself.

Tensor names: `embed`, `pos`, `l<i>.{norm1,norm1b,norm2,norm2b}`, `l<i>.mix.{dq,dq.norm,uq,dkv,dkv.norm,uk,uv,g,o}` or
`l<i>.mix.{q,k,v,o}` with `.b` biases and `.conv` taps and `l<i>.mix.{r1,r2,pb}`, `l<i>.mlp.{router, correction, e<k>.{gate,up,down}}`,
`final.norm`. They have no common root.
"""
from __future__ import annotations

from ..config.ditalorn import DitalornConfig
from ..parts.plan import LayerPlan, ModelPlan, PartSpec, ScheduleEntry
from ..registry import register_architecture

GROUP_TOP = 2   # a group of experts is scored by the sum of its two largest choice scores


def ditalorn_plan(c: DitalornConfig) -> ModelPlan:
    def norm(name):
        return PartSpec("rmsnorm", {"name": name, "size": c.width, "eps": c.norm_eps, "unit_offset": True})

    layers, ignored = [], []
    for i, l in enumerate(c.layers):
        m, p = l.mixer, f"l{i}"
        if l.type == "latent_attention":
            mixer = PartSpec("latent_attention", {
                "prefix": f"{p}.mix", "hidden": c.width, "heads": m.heads, "dim": m.dim, "rot_dim": 0, "vdim": m.vdim, "kv_rank": m.kv_rank, "scale": m.scale,
                "norm_eps": c.norm_eps, "position": PartSpec("none"), "window": m.window, "q_rank": m.q_rank, "gate": True})
        else:
            mixer = PartSpec("sigmoid_attention", {
                "prefix": f"{p}.mix", "hidden": c.width, "heads": m.heads, "kv_heads": m.kv_heads, "dim": m.dim, "vdim": m.vdim, "scale": m.scale,
                "norm_eps": c.norm_eps, "taps": m.conv, "q_temp": m.q_temp})
        params = [("post_mixer_norm", norm(f"{p}.norm1b"))]
        if l.mlp is None:
            ff, ff_norm = PartSpec("none"), PartSpec("none")
            ignored += [f"{p}.norm2", f"{p}.norm2b"]
        else:
            f = l.mlp
            ff_norm = norm(f"{p}.norm2")
            params.append(("post_feed_forward_norm", norm(f"{p}.norm2b")))
            ff = PartSpec("routed_experts", {"prefix": f"{p}.mlp", "hidden": c.width, "expert_ff": f.ff, "experts": f.experts, "top": f.top, "groups": f.groups,
                                             "groups_keep": f.groups_keep, "score": "sigmoid", "correction": "correction", "group_top": GROUP_TOP})
        layers.append(LayerPlan(prefix=p, block="sandwich", mixer=mixer, feed_forward=ff, mixer_norm=norm(f"{p}.norm1"), feed_forward_norm=ff_norm,
                                block_params=tuple(params)))
    return ModelPlan(
        architecture="Ditalorn", vocab_size=c.vocab, hidden_size=c.width, max_positions=c.max_positions,
        embedding=PartSpec("table", {"name": "embed", "vocab": c.vocab, "hidden": c.width, "scale": c.embedding_scale, "positions": "pos",
                                     "max_positions": c.max_positions}),
        layers=tuple(layers), schedule=tuple(ScheduleEntry(i) for i in range(len(layers))),
        final_norm=norm("final.norm"),
        head=PartSpec("linear", {"name": "head", "vocab": c.vocab, "hidden": c.width, "tied_to": "embed"}),
        ignored_tensors=tuple(ignored), root="",
    )


register_architecture(["Ditalorn", "ditalorn"], DitalornConfig.from_dict, ditalorn_plan,
                      traits={"attention": "latent+sigmoid", "qk_norm": False, "norm": "rmsnorm", "norm_unit_offset": True, "rope_style": "none", "activation": "swiglu"})
