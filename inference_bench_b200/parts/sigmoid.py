"""Causal attention whose weights are sigmoids instead of a softmax, behind a short convolution of its projections.

With h the layer's input, p a token's position, H query heads on G key/value heads (query head a uses key/value head a // (H / G)):
    u = [Wq h + bq | Wk h + bk | Wv h + bv]                                   (one product; biases optional)
    y_t = sum_j w[:, j] * u_(t - taps + 1 + j) per channel                    (a causal convolution over time, zeros before the request's start)
    q = y_q * (1 + coef * ln(floor((p + 1) / every) + 1))                     (`q_temp`: a temperature that grows with the position)
    v = y_v / sqrt(mean(y_v^2) + eps) per head                                (`value_norm`; cached so),    k = y_k
    s_ij = (q_i . k_j) * scale - r1_a * ln(1 + r2_a * (i - j)) + pb_a         (`distance_bias`: r1, r2 a head; `score_bias`: pb a head)
    o_i = sum_{j <= i} sigmoid(s_ij) v_j;      out = Wo [o_1 | o_2 | ...] + bo
The weights are not normalised over the keys. There is no rotation: positions enter through the temperature and the distance bias alone.
Every variant is a constructor parameter. The cache holds k and the normed v in pages; the last taps - 1 rows of u are state of the request
(a fixed-size float32 slot). Everything between the projection's float32 sums and the cache, and the scores, the bias and the sigmoid, are
float32; the two products of the attention read bfloat16 operands in the tensor-core kernel (`csrc/sigmoid_attention.cu`).
"""
from __future__ import annotations

from typing import Optional

import numpy as np
import torch

from ..kernels import ops
from . import base
from .base import FixedState, PagedKV, Several, WeightSpec


@base.register_mixer("sigmoid_attention")
class SigmoidAttention(base.Mixer):
    NAMES = ("q", "k", "v", "o", "{}.b", "{}.conv", "r1", "r2", "pb")

    def __init__(self, prefix: str, hidden: int, heads: int, kv_heads: int, dim: int, vdim: int, scale: float, norm_eps: float, taps: int = 1,
                 q_temp: Optional[tuple] = None, value_norm: bool = True, distance_bias: bool = True, score_bias: bool = True, bias: bool = True,
                 names: tuple = NAMES):
        """taps: length of the convolution (0: none at all; 1: one weight a channel and no state). q_temp: (coef, every) or None."""
        if heads <= 0 or kv_heads <= 0 or heads % kv_heads:
            raise ValueError(f"{heads} query heads are not a positive multiple of {kv_heads} kv heads")
        if min(dim, vdim) <= 0 or max(dim, vdim) > 256 or taps < 0:
            raise ValueError(f"head sizes {dim} and {vdim} must be positive and at most 256, taps {taps} not negative")
        if q_temp is not None and int(q_temp[1]) <= 0:
            raise ValueError(f"the query temperature's period must be positive, got {q_temp[1]}")
        self.prefix, self.hidden, self.heads, self.kv_heads, self.dim, self.vdim = prefix, hidden, heads, kv_heads, dim, vdim
        self.scale, self.norm_eps, self.taps = float(scale), float(norm_eps), int(taps)
        self.q_temp = None if q_temp is None else (float(q_temp[0]), int(q_temp[1]))
        self.value_norm, self.distance_bias, self.score_bias, self.bias, self.names = bool(value_norm), bool(distance_bias), bool(score_bias), bool(bias), tuple(names)
        self.row = (heads + kv_heads) * dim + kv_heads * vdim     # channels of u
        self.wqkv = self.wo = self.qkv_bias = self.conv_w = self.r1 = self.r2 = self.pb = None

    def cache_need(self):
        pages = PagedKV(self.kv_heads, max(self.dim, self.vdim))   # one row size for keys and values: the larger of the two
        return Several((pages, FixedState((self.taps - 1, self.row), torch.float32))) if self.taps > 1 else pages

    def _n(self, i: int) -> str:
        return f"{self.prefix}.{self.names[i]}"

    def _of(self, i: int, pattern: int) -> str:
        """A bias or the convolution of matrix i: the matrix's name in that pattern."""
        return f"{self.prefix}.{self.names[pattern].format(self.names[i])}"

    def weight_specs(self):
        sizes = [self.heads * self.dim, self.kv_heads * self.dim, self.kv_heads * self.vdim]
        specs = [WeightSpec(self._n(i), (sizes[i], self.hidden)) for i in range(3)] + [WeightSpec(self._n(3), (self.hidden, self.heads * self.vdim))]
        if self.bias:
            specs += [WeightSpec(self._of(i, 4), (sizes[i],), std=0.1) for i in range(3)] + [WeightSpec(self._of(3, 4), (self.hidden,), std=0.1)]
        if self.taps >= 1:
            specs += [WeightSpec(self._of(i, 5), (sizes[i], self.taps), std=0.5) for i in range(3)]
        if self.distance_bias:
            specs += [WeightSpec(self._n(6), (self.heads,), role="unit"), WeightSpec(self._n(7), (self.heads,), role="unit")]
        if self.score_bias:
            specs.append(WeightSpec(self._n(8), (self.heads,), std=0.5))
        return specs

    def bind(self, weights, rt):
        self.wqkv = rt.matrix(torch.cat([weights[self._n(i)] for i in range(3)], dim=0))
        self.wo = rt.matrix(weights[self._n(3)])
        if self.bias:
            self.qkv_bias = rt.vector(torch.cat([weights[self._of(i, 4)].to(torch.float32) for i in range(3)]))
            self.out_bias = rt.vector(weights[self._of(3, 4)])
        if self.taps >= 1:
            # stored [channel, tap]; the kernel reads a tap's weights for neighbouring channels together: [tap, channel]
            self.conv_w = rt.vector(torch.cat([weights[self._of(i, 5)].to(torch.float32) for i in range(3)], dim=0).t())
        if self.distance_bias:
            self.r1, self.r2 = rt.vector(weights[self._n(6)]), rt.vector(weights[self._n(7)])
        if self.score_bias:
            self.pb = rt.vector(weights[self._n(8)])

    # ------------------------------------------------------------ how a step's work is cut
    def _tensor_cores(self, rt) -> bool:
        how = rt.options.sigmoid_attention
        if how == "generic" or rt.act_dtype != torch.bfloat16:
            return False
        fits = ops.sigmoid_attention_mma_supports(self.heads, self.kv_heads, self.dim, self.vdim) and max(self.dim, self.vdim) % 8 == 0
        if how == "mma" and not fits:
            raise ValueError(f"sigmoid_attention = \"mma\" needs head sizes that are multiples of 16 and at most 16 heads a kv head, got {self.heads}/{self.kv_heads} heads of {self.dim} and {self.vdim}")
        return fits

    def _slices(self, ctx, view, tc: bool) -> tuple[int, int]:
        """(slices, keys per slice): a step of single decoded tokens has few (token, head) pairs, so each one's keys are cut until the GPU is full;
        a step with prompt portions has enough rows. The cut depends on the step's sizes (and, outside a captured step, its longest context) only."""
        key = ("sigmoid slices", self.heads, self.kv_heads, tc)
        if key not in ctx.memo:
            out = (1, 1 << 30)
            if tc and not ctx.fixed_shape and ctx.max_segment_len > 1:
                # prompt portions on the tensor cores: a CTA holds 64 rows and walks their keys in order, so a long context makes a few long chains;
                # up to eight slices of at least 512 keys side by side shorten them while the step has fewer CTAs than four an SM
                longest = int(np.max(ctx.h_positions)) + 1
                ctas = -(-ctx.n_tokens * self.heads // 64)
                if longest > 1024 and ctas < 4 * ctx.rt.sm_count and max(self.dim, self.vdim) <= 128:
                    n = min(8, -(-longest // 512))
                    per = -(-(-(-longest // n)) // 64) * 64
                    out = (-(-longest // per), per)
            elif ctx.fixed_shape or ctx.max_segment_len == 1:
                max_keys = view.table_stride * view.page_size if ctx.fixed_shape else int(np.max(ctx.h_positions)) + 1
                ctas = ctx.n_tokens * self.kv_heads if tc else -(-ctx.n_tokens * self.heads // 4)
                n = max(1, min(2 * ctx.rt.sm_count // max(ctas, 1), -(-max_keys // 128)))
                if n > 1:
                    per = -(-(-(-max_keys // n)) // 64) * 64
                    out = (-(-max_keys // per), per)
            ctx.memo[key] = out
        return ctx.memo[key]

    def _units(self, ctx, per: int):
        """Runs of up to `per` consecutive tokens of one request, int32 [n, 2] of (first token, tokens) on the device; None when every token is its own."""
        if per <= 1 or ctx.fixed_shape or ctx.max_segment_len == 1:
            return None
        key = ("sigmoid units", per)
        if key not in ctx.memo:
            runs = []
            for a, b in zip(ctx.h_seg_start[:-1].tolist(), ctx.h_seg_start[1:].tolist()):
                runs += [(t, min(per, b - t)) for t in range(a, b, per)]
            ctx.memo[key] = torch.tensor(runs, dtype=torch.int32).pin_memory().to(ctx.rt.device, non_blocking=True)
        return ctx.memo[key]

    # ------------------------------------------------------------ one step
    def forward(self, ctx, h, cache):
        rt, T = ctx.rt, ctx.n_tokens
        pages, state = (cache[0], cache[1].tensor) if self.taps > 1 else (cache, None)
        proj = rt.linear(h, self.wqkv)                                       # [P, T, row] = u without its bias
        q = rt.empty((T, self.heads * self.dim))
        ops.qkv_conv(proj, self.qkv_bias, self.conv_w, state, ctx.seg_of_token, ctx.seg_start, ctx.seg_slot, ctx.n_segments, ctx.positions, q, pages, self.heads,
                     self.dim, self.vdim, rt.status, q_temp=self.q_temp, v_norm=self.value_norm, eps=self.norm_eps,
                     single_tokens=ctx.fixed_shape or ctx.n_segments == T)
        tc = self._tensor_cores(rt)
        n_slices, slice_keys = self._slices(ctx, pages.c_view(), tc)
        part = None
        if n_slices > 1:
            skey = ("sigmoid scratch", self.heads, self.vdim, n_slices)
            if skey not in ctx.memo:
                ctx.memo[skey] = rt.empty((T * self.heads * n_slices * self.vdim,), torch.float32)
            part = ctx.memo[skey]
        out = rt.empty((T, self.heads * self.vdim))
        rows, units = 16, None
        if tc:   # a prompt portion: up to 64 rows a CTA (the group's heads of consecutive tokens) share every key and value tile
            group = self.heads // self.kv_heads
            rows = ops.sigmoid_attention_mma_rows(self.dim, self.vdim, group * (1 if ctx.fixed_shape else ctx.max_segment_len))
            units = self._units(ctx, rows // group)
        ops.sigmoid_attention(q, pages, ctx.positions, ctx.seg_of_token, self.scale, self.r1, self.r2, self.pb, out, self.heads, self.dim, self.vdim, rt.status,
                              n_slices=n_slices, slice_keys=slice_keys, part=part, units=units, tensor_cores=tc, rows=rows)
        return rt.linear(out, self.wo)
