"""A feed-forward of routed experts: every token runs through a few of many small gated feed-forwards, chosen by a router,
plus (optionally) one shared expert that every token uses.

    s = softmax(Wr h) over all experts (float32);  experts lie in `groups` equal groups of neighbours, a group's score is its
    largest s, the best `groups_keep` groups stay;  of their experts the `top` with the largest s are chosen;
    out = sum_e weight_e * down_e(silu(gate_e h) * up_e h)  [+ shared(h)],   weight_e = s_e * route_scale
    (with `renorm`: s_e / sum of the chosen s, times route_scale).
`score="sigmoid"`: s_e = sigmoid of expert e's own logit instead of the softmax. `correction` names a tensor of one number an expert
that is added to s where groups and experts are chosen and left out of the weights; `group_top` n makes a group's score the sum of
its n largest choice scores (experts of groups that do not stay cannot be chosen, whatever the sign of their scores). `weight_on="input"`: the weight scales what the expert
reads, out = sum_e down_e(silu(gate_e (weight_e h)) * up_e (weight_e h)), which is not the same thing for a gated expert.
The step's (token, expert) pairs are regrouped by expert on the device (no trip to the host, so the step can be captured),
the experts' products run on the regrouped rows, and the weighted sum returns them to token order.
"""
from __future__ import annotations

import torch

from ..kernels import gemm_tcgen05 as G
from ..kernels import ops
from . import base
from .base import WeightSpec


@base.register_feed_forward("routed_experts")
class RoutedExperts(base.FeedForward):
    def __init__(self, prefix: str, hidden: int, expert_ff: int, experts: int, top: int, route_scale: float = 1.0, groups: int = 1, groups_keep: int = 1,
                 shared_ff: int = 0, renorm: bool = False, names: tuple = ("router", "e{}", "shared", "gate", "up", "down"), score: str = "softmax",
                 weight_on: str = "output", correction: str = "", group_top: int = 1):
        if not 0 < top <= experts or experts % groups or not 0 < groups_keep <= groups:
            raise ValueError(f"top {top} of {experts} experts in {groups} groups of which {groups_keep} stay")
        if score not in ("softmax", "sigmoid") or weight_on not in ("output", "input"):
            raise ValueError(f"score {score!r} (softmax, sigmoid) or weight_on {weight_on!r} (output, input) is not known")
        if not 1 <= group_top <= 4:
            raise ValueError(f"a group's score is the sum of its {group_top} largest scores: 1 to 4 are built")
        self.score, self.weight_on, self.correction, self.group_top = score, weight_on, correction, int(group_top)
        self.w_correction = None
        self.prefix, self.hidden, self.expert_ff, self.experts, self.top = prefix, hidden, expert_ff, experts, top
        self.route_scale, self.groups, self.groups_keep, self.shared_ff, self.renorm, self.names = route_scale, groups, groups_keep, shared_ff, renorm, tuple(names)
        self.w_router = self.w_gu = self.w_d = self.shared_gu = self.shared_d = None

    def _expert(self, k: int, which: int) -> str:
        return f"{self.prefix}.{self.names[1].format(k)}.{self.names[3 + which]}"

    def _shared(self, which: int) -> str:
        return f"{self.prefix}.{self.names[2]}.{self.names[3 + which]}"

    def weight_specs(self):
        W, F = self.hidden, self.expert_ff
        specs = [WeightSpec(f"{self.prefix}.{self.names[0]}", (self.experts, W))]
        for k in range(self.experts):
            specs += [WeightSpec(self._expert(k, 0), (F, W)), WeightSpec(self._expert(k, 1), (F, W)), WeightSpec(self._expert(k, 2), (W, F))]
        if self.correction:
            specs.append(WeightSpec(f"{self.prefix}.{self.correction}", (self.experts,), std=0.1))
        if self.shared_ff:
            S = self.shared_ff
            specs += [WeightSpec(self._shared(0), (S, W)), WeightSpec(self._shared(1), (S, W)), WeightSpec(self._shared(2), (W, S))]
        return specs

    def bind(self, weights, rt):
        self.w_router = rt.matrix(weights[f"{self.prefix}.{self.names[0]}"])
        if self.correction:
            self.w_correction = rt.vector(weights[f"{self.prefix}.{self.correction}"])
        # [experts, gate rows then up rows, width] and [experts, width, inner]: one tensor each, so a tile of the grouped product finds its expert by an offset
        self.w_gu = rt.upload(torch.stack([torch.cat([weights[self._expert(k, 0)], weights[self._expert(k, 1)]], dim=0) for k in range(self.experts)]), rt.act_dtype)
        self.w_d = rt.upload(torch.stack([weights[self._expert(k, 2)] for k in range(self.experts)]), rt.act_dtype)
        if self.shared_ff:
            self.shared_gu = rt.matrix(torch.cat([weights[self._shared(0)], weights[self._shared(1)]], dim=0))
            self.shared_d = rt.matrix(weights[self._shared(2)])

    def forward(self, ctx, h):
        rt, T, E, top = ctx.rt, ctx.n_tokens, self.experts, self.top
        R = T * top
        logits = rt.linear(h, self.w_router)                     # float32 partial sums [P, T, E]
        idx, wt = rt.empty((T, top), torch.int32), rt.empty((T, top), torch.float32)
        ops.moe_route(logits, self.groups, self.groups_keep, top, self.route_scale, self.renorm, idx, wt, self.score, correction=self.w_correction, group_top=self.group_top)
        on_input = self.weight_on == "input"
        offsets, tile_start = rt.empty((E + 1,), torch.int32), rt.empty((E + 1,), torch.int32)
        row_of_pair, token_of_row = rt.empty((R,), torch.int32), rt.empty((R,), torch.int32)
        how = rt.options.expert_gemm
        bn = G.grouped_token_tile(R, E, self.expert_ff, rt.sm_count)
        act = rt.empty((R, self.expert_ff))
        y = rt.empty((R, self.hidden), torch.float32)
        if how in ("auto", "tcgen05") and rt.act_dtype == torch.bfloat16 and rt.gemm != "simt" and G.grouped_supported(self.hidden, self.expert_ff, bn):
            # the tcgen05 kernel of the single-matrix products, its tiles taking their expert from the tile table
            ops.moe_sort(idx, E, offsets, tile_start, row_of_pair, token_of_row, tile_rows=bn)
            xs = rt.empty((R, self.hidden))
            if on_input:
                ops.scatter_scaled_rows(h, row_of_pair, wt, xs)
            else:
                ops.gather_rows(h, token_of_row, xs)
            G.gemm_grouped_swiglu(xs, self.w_gu, act, bn, offsets, tile_start, rt.status)
            G.gemm_grouped(act, self.w_d, y, bn, offsets, tile_start, rt.status)
        else:
            if how == "tcgen05":
                raise ValueError(f"expert_gemm = \"tcgen05\" needs bfloat16 and inner sizes that are multiples of 8 (of 64 for few tokens), got {self.hidden} and {self.expert_ff}")
            tc = how != "simt"
            ops.moe_sort(idx, E, offsets, tile_start, row_of_pair, token_of_row)
            src, rows = h, token_of_row
            if on_input:   # the rows in the experts' order, each times its weight; the product then reads them as they lie
                src, rows = rt.empty((R, self.hidden)), None
                ops.scatter_scaled_rows(h, row_of_pair, wt, src)
            ops.gemm_grouped(src, rows, self.w_gu, act, offsets, tile_start, gated=True, tensor_cores=tc and ops.rows_mma_fits(src, self.w_gu))
            ops.gemm_grouped(act, None, self.w_d, y, offsets, tile_start, gated=False, tensor_cores=tc and ops.rows_mma_fits(act, self.w_d))
        shared = rt.linear(rt.gate_up_act(h, self.shared_gu), self.shared_d) if self.shared_ff else None
        out = rt.empty((1, T, self.hidden), torch.float32)
        ops.moe_combine(y, row_of_pair, wt, shared, out[0], weighted=not on_input)
        return out
