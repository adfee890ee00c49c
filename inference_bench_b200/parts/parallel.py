"""Mixers that run side by side on the same input and are summed with fixed weights: out = sum_b scale_b * branch_b(h).

All branches' input projections are one matrix product (their rows concatenated; every branch reads its own columns of the float32
sums), and all output projections are one product too: every branch writes scale_b times what its output projection reads into its
columns of one buffer, and the projections' matrices are concatenated along their inputs. A branch's output bias times its scale is
the mixer's `out_bias`.

Two branches exist:

"chunk_attention": grouped-query attention whose values are its keys as projected (there is no value projection); q and k have biases,
are rotated over the first `rotary_dim` entries of a head and then divided by their root mean square over the head (no weights);
score = q.k * scale; a position sees the earlier positions of its own block of `chunk` positions, counted from the request's position
0; the softmax's denominator also holds exp(sink_head), a learned number per head without key or value; head a's output is multiplied
by sigmoid(W_g h)_a. Keys (rotated, normed) and values (the keys as projected) live in the paged cache. bfloat16 heads of 64 or 128 run on
the tensor-core kernels (prompt portions on the flash kernel, decoded tokens on the split-context kernels: blocks of positions are their
negative window, the sink's scores, the gate and the branch's scale their output tail); everything else on the generic kernel.

"decayed_linear": per head S <- decay_head S + k v^T, o = S^T q with q, k, v = silu of their projections and S [dim, vdim] float32 state of
the request; all heads' o are normed together (RMS norm with a weight), multiplied by sigmoid(W_g h) elementwise and projected.
Long segments go through the recurrence kernel's chunked form (parts/recurrent.py).
"""
from __future__ import annotations

from typing import Optional

import torch

from ..kernels import ops
from . import base
from .base import FixedState, PagedKV, Several, WeightSpec
from .plan import PartSpec
from .recurrent import GatedLinearRecurrence


class ChunkAttentionBranch:
    def __init__(self, prefix: str, hidden: int, heads: int, kv_heads: int, head_dim: int, chunk: int, scale: float, norm_eps: float,
                 position: base.PositionEncoding, names: tuple = ("q", "k", "sink", "g", "o", "{}.b")):
        if heads <= 0 or kv_heads <= 0 or heads % kv_heads:
            raise ValueError(f"{heads} query heads are not a positive multiple of {kv_heads} kv heads")
        if head_dim <= 0 or head_dim % 2 or head_dim > 256:
            raise ValueError(f"head size {head_dim} must be even, positive and at most 256")
        if chunk <= 0:
            raise ValueError(f"the block of positions {chunk} must be positive")
        if getattr(position, "pairing", "half") != "half":
            raise ValueError("this attention turns entry i with i + rotary_dim/2: it needs a position encoding with pairing=\"half\"")
        self.prefix, self.hidden, self.heads, self.kv_heads, self.head_dim = prefix, hidden, heads, kv_heads, head_dim
        self.chunk, self.scale, self.norm_eps, self.position, self.names = chunk, float(scale), norm_eps, position, tuple(names)
        self.sink = None

    # what the parallel mixer asks of a branch
    @property
    def in_rows(self) -> int:
        return (self.heads + self.kv_heads) * self.head_dim + self.heads     # [q | k | g]

    @property
    def out_cols(self) -> int:
        return self.heads * self.head_dim

    def cache_need(self):
        return PagedKV(self.kv_heads, self.head_dim, None)

    def _n(self, i: int) -> str:
        return f"{self.prefix}.{self.names[i]}"

    def _b(self, i: int) -> str:
        return f"{self.prefix}.{self.names[5].format(self.names[i])}"

    def weight_specs(self):
        hd = self.head_dim
        return [WeightSpec(self._n(0), (self.heads * hd, self.hidden)), WeightSpec(self._b(0), (self.heads * hd,), std=0.1),
                WeightSpec(self._n(1), (self.kv_heads * hd, self.hidden)), WeightSpec(self._b(1), (self.kv_heads * hd,), std=0.1),
                WeightSpec(self._n(2), (self.heads,), std=1.0), WeightSpec(self._n(3), (self.heads, self.hidden)),
                WeightSpec(self._n(4), (self.hidden, self.heads * hd)), WeightSpec(self._b(4), (self.hidden,), std=0.1)]

    def in_matrix(self, weights):
        return [weights[self._n(0)], weights[self._n(1)], weights[self._n(3)]]

    def in_bias(self, weights):
        f = torch.float32
        return [weights[self._b(0)].to(f), weights[self._b(1)].to(f), torch.zeros(self.heads, dtype=f, device=weights[self._b(0)].device)]

    def out_matrix(self, weights):
        return weights[self._n(4)]

    def out_bias(self, weights) -> Optional[torch.Tensor]:
        return weights[self._b(4)]

    def bind(self, weights, rt):
        self.sink = rt.vector(weights[self._n(2)])
        self.position.bind(weights, rt)

    def run(self, ctx, proj, col0: int, bias, cache, out, out_col: int, scale: float) -> None:
        rt, hd = ctx.rt, self.head_dim
        if out_col != 0:
            raise RuntimeError("the attention branch writes the first columns of the output buffer: it must be the first branch")
        cos, sin = self.position.tables(ctx)
        q = rt.empty((ctx.n_tokens, self.heads * hd))
        q_col, k_col, g_col = col0, col0 + self.heads * hd, col0 + (self.heads + self.kv_heads) * hd
        ops.qk_norm_rope_kv(proj, None, None, self.norm_eps, cos, sin, ctx.positions, ctx.seg_of_token, q, cache, self.heads, rt.status, bias=bias,
                            qk_dim=hd, v_dim=hd, columns=(q_col, k_col, None), unit_norm_after=True)
        from ..kernels import attention
        attention.paged_attention(ctx, q, cache, self.heads, None, self.scale, qk_dim=hd, v_dim=hd, sink=True, chunk=self.chunk, sink_values=self.sink,
                                  gate=(proj, g_col), out_scale=scale, out=out)


class DecayedLinearBranch:
    def __init__(self, prefix: str, hidden: int, heads: int, dim: int, vdim: int, decay, norm_eps: float, names: tuple = ("q", "k", "v", "g", "norm", "o")):
        decay = tuple(float(d) for d in decay)
        if heads <= 0 or dim <= 0 or vdim <= 0 or dim > 512:
            raise ValueError(f"heads {heads}, dim {dim} (at most 512) and vdim {vdim} must be positive")
        if len(decay) != heads or any(not 0.0 <= d <= 1.0 for d in decay):
            raise ValueError(f"{heads} heads need {heads} decays in [0, 1], got {decay}")
        self.prefix, self.hidden, self.heads, self.dim, self.vdim, self.decay, self.norm_eps, self.names = prefix, hidden, heads, dim, vdim, decay, norm_eps, tuple(names)
        self.decay_dev = self.norm_w = None

    @property
    def in_rows(self) -> int:
        return 2 * self.heads * self.dim + 2 * self.heads * self.vdim      # [q | k | v | g]

    @property
    def out_cols(self) -> int:
        return self.heads * self.vdim

    def cache_need(self):
        return FixedState((self.heads, self.dim, self.vdim), torch.float32)

    def _n(self, i: int) -> str:
        return f"{self.prefix}.{self.names[i]}"

    def weight_specs(self):
        H, D, V = self.heads, self.dim, self.vdim
        return [WeightSpec(self._n(0), (H * D, self.hidden)), WeightSpec(self._n(1), (H * D, self.hidden)), WeightSpec(self._n(2), (H * V, self.hidden)),
                WeightSpec(self._n(3), (H * V, self.hidden)), WeightSpec(self._n(4), (H * V,), role="norm"), WeightSpec(self._n(5), (self.hidden, H * V))]

    def in_matrix(self, weights):
        return [weights[self._n(i)] for i in range(4)]

    def in_bias(self, weights):
        return None

    def out_matrix(self, weights):
        return weights[self._n(5)]

    def out_bias(self, weights):
        return None

    def bind(self, weights, rt):
        self.decay_dev = rt.upload(torch.tensor(self.decay, dtype=torch.float32))
        self.norm_w = rt.vector(weights[self._n(4)])

    def run(self, ctx, proj, col0: int, bias, cache, out, out_col: int, scale: float) -> None:
        rt, H, D, V = ctx.rt, self.heads, self.dim, self.vdim
        o = rt.empty((ctx.n_tokens, H, V), torch.float32)
        short, long_segs, chunks = GatedLinearRecurrence._cut(ctx)
        ops.gated_recurrence(proj, None, self.decay_dev, cache.tensor, ctx.seg_start, ctx.seg_slot, ctx.n_segments, o, H, D, V, seg_list=short, long_segs=long_segs,
                             chunks=chunks, fixed_decay=True, columns=(col0, col0 + H * D, col0 + 2 * H * D))
        ops.gated_rmsnorm(o.view(ctx.n_tokens, H * V), self.norm_w, self.norm_eps, proj, col0 + 2 * H * D + H * V, scale, out, out_col)


BRANCHES = {"chunk_attention": ChunkAttentionBranch, "decayed_linear": DecayedLinearBranch}


@base.register_mixer("parallel")
class ParallelMixer(base.Mixer):
    def __init__(self, hidden: int, branches: tuple):
        """branches: ((kind, scale, params), ...): the branch's kind (`BRANCHES`), its weight in the sum and its constructor's parameters (a
        `position` among them may be a position encoding already built)."""
        self.hidden = hidden
        self.branches, self.scales = [], []
        for kind, scale, params in branches:
            if kind not in BRANCHES:
                raise KeyError(f"no branch of kind {kind!r} (known: {', '.join(sorted(BRANCHES))})")
            params = dict(params)
            if isinstance(params.get("position"), PartSpec):
                params["position"] = base.make(base.POSITION_ENCODINGS, "position encoding", params["position"].kind, **params["position"].params)
            self.branches.append(BRANCHES[kind](hidden=hidden, **params))
            self.scales.append(float(scale))
        if not self.branches:
            raise ValueError("a parallel mixer needs a branch")
        self.w_in = self.w_out = self.in_bias = None
        self.in_cols, self.out_cols = [], []
        a = b = 0
        for br in self.branches:
            self.in_cols.append(a)
            self.out_cols.append(b)
            a, b = a + br.in_rows, b + br.out_cols
        self.in_rows, self.out_width = a, b

    def cache_need(self):
        return Several(tuple(br.cache_need() for br in self.branches))

    def weight_specs(self):
        return [s for br in self.branches for s in br.weight_specs()]

    def bind(self, weights, rt):
        rows, bias, any_bias = [], [], False
        for br in self.branches:
            m = br.in_matrix(weights)
            rows += m
            b = br.in_bias(weights)
            any_bias = any_bias or b is not None
            bias += b if b is not None else [torch.zeros(sum(x.shape[0] for x in m), dtype=torch.float32, device=m[0].device)]
        self.w_in = rt.matrix(torch.cat(rows, dim=0))
        self.in_bias = rt.vector(torch.cat(bias)) if any_bias else None
        self.w_out = rt.matrix(torch.cat([br.out_matrix(weights) for br in self.branches], dim=1))
        out_bias = None
        for br, s in zip(self.branches, self.scales):
            b = br.out_bias(weights)
            if b is not None:
                out_bias = s * b.to(torch.float32) if out_bias is None else out_bias + s * b.to(torch.float32)
            br.bind(weights, rt)
        self.out_bias = None if out_bias is None else rt.vector(out_bias)

    def forward(self, ctx, h, cache):
        rt = ctx.rt
        proj = rt.linear(h, self.w_in)                                   # [P, T, all branches' rows]
        out = rt.empty((ctx.n_tokens, self.out_width))
        for br, s, c_in, c_out, view in zip(self.branches, self.scales, self.in_cols, self.out_cols, cache):
            br.run(ctx, proj, c_in, self.in_bias, view, out, c_out, s)
        return rt.linear(out, self.w_out)
