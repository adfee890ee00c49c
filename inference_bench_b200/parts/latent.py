"""Latent attention: keys and values of all heads are linear maps of one small latent per token, and only that latent
and one rotated key part shared by the heads are cached.

With h the layer's input, per token:
    q = Wq h, per head [q_n (dim) | q_r (rot_dim)];   [c_raw (kv_rank) | r_raw (rot_dim)] = Wdkv h;
    c = w_c * c_raw / rms(c_raw),  r = turn(r_raw),  q_r <- turn(q_r)      (pairs 2i, 2i+1; angle pos * base^(-2i/dims))
    head a:  k = Wuk_a c,  v = Wuv_a c,  s_j = (q_n . k_j + q_r . r_j) * scale  over j <= own position,  o_a = sum_j softmax(s)_j v_j
    out = Wo [o_1 | o_2 | ...]
The cache row of a token is [c | r]. The kernels never build k and v: q_n . (Wuk_a c) = (Wuk_a^T q_n) . c and
sum_j p_j Wuv_a c_j = Wuv_a (sum_j p_j c_j), so a head's query becomes [Wuk_a^T q_n | q_r] against the cached rows, and the
weighted sum of latents goes through Wuv_a afterwards (two small per-head products around one attention kernel that reads
kv_rank + rot_dim values a key for all heads together). A layer with own_kv=False has no Wdkv and reads the rows another
layer cached.

Variants, each a constructor parameter. `q_rank` n: the queries go through a latent of their own, c_q = w_q * rms_unit(Wdq h) (n values),
q = Wuq c_q; the layer's first product is then [Wdq | Wdkv] h and a second one makes the heads' queries. `window` W: a position sees
itself and the W - 1 positions before it (the cache then keeps only those pages). `gate`: head a's output is multiplied by
sigmoid(Wg h)_a, one number a head from the layer's input (its rows ride in the first product; the sigmoid sits in the epilogue of the
per-head product with Wuv). rot_dim 0: no rotated part at all (the position encoding is then "none").
"""
from __future__ import annotations

from typing import Optional

import numpy as np
import torch

from ..kernels import ops
from . import base
from .base import PagedRows, WeightSpec


@base.register_mixer("latent_attention")
class LatentAttention(base.Mixer):
    def __init__(self, prefix: str, hidden: int, heads: int, dim: int, rot_dim: int, vdim: int, kv_rank: int, scale: float, norm_eps: float,
                 position: base.PositionEncoding, own_kv: bool = True, window: Optional[int] = None,
                 names: tuple = ("q", "dkv", "dkv.norm", "uk", "uv", "o", "dq", "dq.norm", "uq", "g"), q_rank: Optional[int] = None, gate: bool = False):
        if getattr(position, "pairing", "interleaved") != "interleaved":
            raise ValueError("latent attention turns entry 2i with 2i + 1: it needs a position encoding with pairing=\"interleaved\" (or none)")
        if window is not None and (window <= 0 or not own_kv):
            raise ValueError("a window must be positive, and a layer that reads another layer's rows takes that layer's window")
        if q_rank is not None and (q_rank <= 0 or not own_kv):
            raise ValueError("a query latent must have a positive size, and is built for layers that keep their own latent")
        self.window, self.q_rank, self.gate = window, q_rank, bool(gate)
        self.w_uq = self.q_norm = None
        self.prefix, self.hidden, self.heads, self.dim, self.rot_dim, self.vdim, self.kv_rank = prefix, hidden, heads, dim, rot_dim, vdim, kv_rank
        self.scale, self.norm_eps, self.position, self.own_kv, self.names = scale, norm_eps, position, own_kv, tuple(names)
        self.w_in = self.wuk_t = self.wuv = self.wo = self.c_norm = None

    def cache_need(self):
        return PagedRows(self.kv_rank + self.rot_dim, self.window) if self.own_kv else None

    def _name(self, i: int) -> str:
        return f"{self.prefix}.{self.names[i]}"

    def weight_specs(self):
        H, r = self.heads, self.kv_rank
        specs = [WeightSpec(self._name(3), (H * self.dim, r)), WeightSpec(self._name(4), (H * self.vdim, r)), WeightSpec(self._name(5), (self.hidden, H * self.vdim))]
        if self.q_rank is None:
            specs.append(WeightSpec(self._name(0), (H * (self.dim + self.rot_dim), self.hidden)))
        else:
            specs += [WeightSpec(self._name(6), (self.q_rank, self.hidden)), WeightSpec(self._name(7), (self.q_rank,), role="norm"),
                      WeightSpec(self._name(8), (H * (self.dim + self.rot_dim), self.q_rank))]
        if self.gate:
            specs.append(WeightSpec(self._name(9), (H, self.hidden)))
        if self.own_kv:
            specs += [WeightSpec(self._name(1), (r + self.rot_dim, self.hidden)), WeightSpec(self._name(2), (r,), role="norm")]
        return specs

    def bind(self, weights, rt):
        H, r = self.heads, self.kv_rank
        rows = [weights[self._name(0) if self.q_rank is None else self._name(6)]]
        if self.own_kv:
            rows.append(weights[self._name(1)])
            self.c_norm = rt.vector(weights[self._name(2)])
        if self.gate:
            rows.append(weights[self._name(9)])
        self.w_in = rt.matrix(torch.cat(rows, dim=0))   # [q of all heads (or the query latent) | latent | key part | gates] rows: one product for the layer's input
        if self.q_rank is not None:
            self.w_uq, self.q_norm = rt.matrix(weights[self._name(8)]), rt.vector(weights[self._name(7)])
        self.wuk_t = rt.upload(weights[self._name(3)].view(H, self.dim, r).transpose(1, 2), rt.act_dtype)   # [H, rank, dim]: q_n -> rank values
        self.wuv = rt.upload(weights[self._name(4)].view(H, self.vdim, r), rt.act_dtype)                    # [H, vdim, rank]
        self.wo = rt.matrix(weights[self._name(5)])
        self.position.bind(weights, rt)

    def _slices(self, ctx, view) -> tuple[int, int]:
        """(slices, keys per slice) of the attention kernel: a step of single decoded tokens has few (token, head block)
        pairs, so each one's keys are cut until every SM has two CTAs; a step with prompt portions has enough rows.
        The cut depends on the step's sizes (and, outside a captured step, its longest context) only."""
        key = ("latent slices", self.heads, self.window)
        if key not in ctx.memo:
            single = ctx.fixed_shape or ctx.max_segment_len == 1
            out = (1, 1 << 30)
            if single:
                max_keys = view.table_stride * view.page_size if ctx.fixed_shape else int(np.max(ctx.h_positions)) + 1
                if self.window is not None:
                    max_keys = min(max_keys, self.window)
                ctas = ctx.n_tokens * -(-self.heads // (16 if self._tensor_cores(ctx.rt) else 8))
                n = max(1, min(ctx.rt.sm_count // ctas, -(-max_keys // 128)))   # two key tiles a slice at least: the second arrives while the first is used
                if n > 1:
                    per = -(-(-(-max_keys // n)) // 64) * 64
                    out = (-(-max_keys // per), per)
            ctx.memo[key] = out
        return ctx.memo[key]

    def _rows_and_units(self, ctx):
        """For the tensor-core kernel: (query rows a CTA holds, runs of consecutive tokens of one request that fill them as int32 [n, 2]
        of (first token, tokens) on the device, or None when every token is a unit of its own)."""
        longest = 1 if ctx.fixed_shape else ctx.max_segment_len
        rows = ops.latent_attention_mma_rows(self.kv_rank, self.kv_rank + self.rot_dim, self.heads * longest)
        per = rows // self.heads
        if per <= 1 or longest == 1:
            return rows, None
        return rows, self._units(ctx, per)

    def _units(self, ctx, per):
        key = ("latent units", per)
        if key not in ctx.memo:
            runs = []
            for a, b in zip(ctx.h_seg_start[:-1].tolist(), ctx.h_seg_start[1:].tolist()):
                runs += [(t, min(per, b - t)) for t in range(a, b, per)]
            ctx.memo[key] = torch.tensor(runs, dtype=torch.int32).pin_memory().to(ctx.rt.device, non_blocking=True)
        return ctx.memo[key]

    def _tensor_cores(self, rt) -> bool:
        how = rt.options.latent_attention
        if how == "generic" or rt.act_dtype != torch.bfloat16:
            return False
        fits = ops.latent_attention_mma_supports(self.kv_rank, self.kv_rank + self.rot_dim)
        if how == "mma" and not fits:
            raise ValueError(f"latent_attention = \"mma\" needs a latent and a rotated part that are multiples of 16 (up to 512 and 576 together), got {self.kv_rank} and {self.rot_dim}")
        return fits

    def forward(self, ctx, h, cache):
        rt, T, H, r, rot = ctx.rt, ctx.n_tokens, self.heads, self.kv_rank, self.rot_dim
        cos, sin = self.position.tables(ctx)
        qd = rt.linear(h, self.w_in)
        q_nope = rt.empty((T, H, self.dim))
        q_full = rt.empty((T, H, r + rot), torch.float32)
        gate = None
        if self.gate:   # the gates' columns are the last of the first product; their sigmoid waits for the product with Wuv
            gate = (qd, qd.shape[2] - H)
        if self.q_rank is None:
            if self.gate:
                raise NotImplementedError("an output gate is built for layers whose queries go through a latent")
            ops.latent_prepare(qd, self.c_norm, self.norm_eps, cos, sin, ctx.positions, ctx.seg_of_token, q_nope, q_full, cache, H, self.dim, rot, r,
                               self.own_kv, rt.status)
        else:
            cq = rt.empty((T, self.q_rank))
            ops.latent_down(qd, self.q_rank, self.q_norm, cq, self.c_norm, self.norm_eps, cos, sin, ctx.positions, ctx.seg_of_token, cache, r, rot, rt.status)
            ops.latent_prepare(rt.linear(cq, self.w_uq), None, self.norm_eps, cos, sin, ctx.positions, ctx.seg_of_token, q_nope, q_full, cache, H, self.dim, rot, r,
                               False, rt.status)
        tc = rt.options.expert_gemm != "simt"   # (the per-head maps have the m16n8k16 kernel and the FMA kernel)
        ops.gemm_heads(q_nope, self.wuk_t, q_full, r, tensor_cores=tc and ops.rows_mma_fits(q_nope, self.wuk_t))
        n_slices, slice_keys = self._slices(ctx, cache.c_view())
        scratch = None
        if n_slices > 1:
            skey = ("latent scratch", H, r, n_slices)
            if skey not in ctx.memo:
                ctx.memo[skey] = (rt.empty((T * H * n_slices * r,), torch.float32), rt.empty((T * H * n_slices * 2,), torch.float32))
            scratch = ctx.memo[skey]
        u = rt.empty((T, H, r))
        if self._tensor_cores(rt):
            rows, units = self._rows_and_units(ctx)
            ops.latent_attention_mma(q_full, cache, ctx.positions, ctx.seg_of_token, units, self.scale, u, r, n_slices, slice_keys, scratch, rt.status, rows, window=self.window)
        else:
            ops.latent_attention(q_full, cache, ctx.positions, ctx.seg_of_token, self.scale, u, r, n_slices, slice_keys, scratch, rt.status, window=self.window)
        v = rt.empty((T, H, self.vdim))
        ops.gemm_heads(u, self.wuv, v, self.vdim, tensor_cores=tc and ops.rows_mma_fits(u, self.wuv), gate=gate)
        return rt.linear(v.view(T, H * self.vdim), self.wo)
