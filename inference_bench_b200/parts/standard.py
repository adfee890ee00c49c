"""The parts the Qwen3 dense decoder is made of, each parametrized by its own sizes and constants.

Formulas follow v0l/inference-bench's `specrt`; the file:line beside each class names where the
reference computes the same thing.
"""
from __future__ import annotations

import math
from typing import Optional

import torch

from ..kernels import ops
from . import base
from .base import FixedState, PagedKV, WeightSpec


# ------------------------------------------------------------------------------------------ norm
@base.register_norm("rmsnorm")
class RMSNorm(base.Norm):
    """y = w * (x * rsqrt(mean(x^2) + eps)), float32 arithmetic, fused with the residual add that
    precedes it (crates/kir/tests/golden/rmsnorm_sm120.cu:19-29; no unit offset for this family,
    crates/specrt/src/weights.rs:877-880)."""

    def __init__(self, name: str, size: int, eps: float, unit_offset: bool = False, scalar: bool = False):
        """unit_offset: the stored weight lies around zero and the scale is 1 + w. scalar: the stored weight is one number for all
        channels (a tensor without axes); the kernels get it as a vector of equal entries."""
        self.name, self.size, self.eps, self.unit_offset, self.scalar = name, size, eps, unit_offset, scalar
        self.w: Optional[torch.Tensor] = None

    def weight_specs(self):
        return [WeightSpec(self.name, () if self.scalar else (self.size,), role="norm_offset" if self.unit_offset else "norm")]

    def bind(self, weights, rt):
        w = weights[self.name]
        self.w = rt.vector(w.reshape(1).expand(self.size) if self.scalar else w)
        if self.unit_offset:
            self.w = self.w + 1.0   # float32, once: the kernels multiply by the scale whatever it was stored as

    def add_normed(self, ctx, x, delta, mult):
        rt = ctx.rt
        act = None if rt.act_dtype == torch.float32 else rt.empty(tuple(x.shape))
        ops.norm_residual(x, delta, self.w, float(mult), self.eps, act)
        return x if act is None else act

    takes_normed_delta = True

    def forward(self, ctx, x, delta, rows=None):
        n = x.shape[0] if rows is None else rows.shape[0]
        out = ctx.rt.empty((n, self.size))
        if isinstance(delta, base.NormedDelta):   # the contribution goes through its own norm on its way into the stream: one kernel for both norms
            post = delta.norm
            if not isinstance(post, RMSNorm) or post.eps != self.eps:
                raise ValueError("a contribution's own norm must be an RMS norm with this norm's epsilon")
            ops.post_norm(x, delta.delta, delta.bias, post.w, self.w, out, self.eps, rows)
            return out
        ops.add_rmsnorm(x, delta, self.w, out, self.eps, rows)
        return out

    def add_post(self, ctx, x, delta, bias, next_norm: Optional["RMSNorm"] = None):
        """This norm on a sublayer's output: x += w * rms_unit(sum of `delta` + bias), in place; with `next_norm`, returns that norm of the
        updated stream in the activation dtype (the next sublayer's input), from the same kernel."""
        out = None if next_norm is None else ctx.rt.empty((x.shape[0], self.size))
        ops.post_norm(x, delta, bias, self.w, None if next_norm is None else next_norm.w, out, self.eps)
        return out


@base.register_norm("layernorm")
class LayerNorm(base.Norm):
    """y = w * (x - mean(x)) / sqrt(mean((x - mean)^2) + eps), no bias, float32 arithmetic, fused with the residual add that precedes
    it. `forward` takes the extras a block may need from that kernel: a per-channel scale and a bias on the contribution it adds, a
    copy of the updated stream, and a layout of the normed rows for a convolution over time (`ops.ConvLayout`; the rows then stay
    float32 and keep their place in that layout)."""

    takes_layout = True   # `forward` takes the extras named above (what a block with input convolutions asks of its norms)

    def __init__(self, name: str, size: int, eps: float):
        self.name, self.size, self.eps = name, size, eps
        self.w: Optional[torch.Tensor] = None

    def weight_specs(self):
        return [WeightSpec(self.name, (self.size,), role="norm")]

    def bind(self, weights, rt):
        self.w = rt.vector(weights[self.name])

    def forward(self, ctx, x, delta, rows=None, delta_scale=None, delta_bias=None, x_copy=None, layout=None):
        if layout is not None:
            out = ctx.rt.empty((layout.rows(x.shape[0]), self.size), torch.float32)
        else:
            out = ctx.rt.empty((x.shape[0] if rows is None else rows.shape[0], self.size))
        ops.add_layernorm(x, delta, self.w, out, self.eps, rows, delta_scale, delta_bias, x_copy, layout)
        return out


# ------------------------------------------------------------------------------------------ position
@base.register_position_encoding("rope")
class RotaryEmbedding(base.PositionEncoding):
    """Half-rotation ("NeoX") rotary encoding over the first `rotary_dim` dims of a head:
    inv_freq_i = theta^(-2i/rotary_dim), angle = float(pos) * inv_freq_i in float32
    (crates/kir/tests/golden/attention/RopeKvWrite_bf16x2_sm120.cu:32-35, 200-206)."""

    def __init__(self, rotary_dim: int, theta: float, pairing: str = "half", scaling: Optional[tuple] = None):
        """pairing: which entries a mixer turns together with these angles: "half" pairs entry i with i + rotary_dim/2,
        "interleaved" pairs entry 2i with 2i + 1. The tables are the same; the mixer's kernel does the pairing.
        scaling: None or (factor, low, high, original): frequencies are rescaled by wavelength l = 2 pi / f in three bands. Where
        l < original / high the frequency stays; where l > original / low it becomes f / factor; between the two it is
        (1 - s) f / factor + s f with s = (original / l - low) / (high - low)."""
        if scaling is not None:
            scaling = tuple(float(v) for v in scaling)
            if len(scaling) != 4 or scaling[0] <= 0 or scaling[2] == scaling[1] or scaling[3] <= 0:
                raise ValueError(f"rotary scaling must be (factor, low, high, original) with high != low, got {scaling}")
        self.scaling = scaling
        if rotary_dim % 2:
            raise ValueError(f"rotary_dim {rotary_dim} must be even")
        if pairing not in ("half", "interleaved"):
            raise ValueError(f"pairing {pairing!r} is not known (half, interleaved)")
        self.rotary_dim, self.theta, self.pairing = rotary_dim, theta, pairing
        self.inv_freq: Optional[torch.Tensor] = None

    def bind(self, weights, rt):
        i = torch.arange(0, self.rotary_dim, 2, dtype=torch.float64)
        f = 1.0 / torch.pow(torch.tensor(self.theta, dtype=torch.float64), i / self.rotary_dim)
        if self.scaling is not None:
            factor, low, high, original = self.scaling
            wavelength = 2.0 * math.pi / f
            blend = (original / wavelength - low) / (high - low)
            mid = (1.0 - blend) * f / factor + blend * f
            f = torch.where(wavelength < original / high, f, torch.where(wavelength > original / low, f / factor, mid))
        self.inv_freq = rt.upload(f.to(torch.float32))

    def tables(self, ctx):
        key = ("rope", self.rotary_dim, self.theta, self.scaling)
        if key not in ctx.memo:
            half = self.rotary_dim // 2
            cos = ctx.rt.empty((ctx.n_tokens, half), torch.float32)
            sin = ctx.rt.empty((ctx.n_tokens, half), torch.float32)
            ops.rope_table(ctx.positions, self.inv_freq, cos, sin)
            ctx.memo[key] = (cos, sin)
        return ctx.memo[key]


@base.register_position_encoding("none")
class NoPositionEncoding(base.PositionEncoding):
    def __init__(self):
        pass

    def tables(self, ctx):
        return None, None


# ------------------------------------------------------------------------------------------ mixer
@base.register_mixer("attention")
class Attention(base.Mixer):
    """Causal grouped-query attention over a paged cache, with optional per-head RMSNorm of q and k
    before the rotation and an optional window.

    qkv = Wqkv h (q, k, v rows concatenated at load: crates/specrt/src/weights.rs:886-953);
    per-head norm then RoPE (crates/kir/src/cuda/attention/common.rs:49-96);
    s = q.k / sqrt(head_dim), keys visible when key <= pos and, with a window W, key > pos - W
    (crates/kir/src/cuda/attention/flash_mma.rs:193); out = Wo (softmax(s) v).
    With own_kv=False the layer has only a q projection and reads the cache it is given.

    Variants, each a constructor parameter: `bias` (q, k, v and the output projection have bias vectors; the output's is handed
    to the block as `out_bias`), `softcap` c (s <- c tanh(s / c) after the scale), `sink` (the softmax's denominator has one added:
    a key of score 0 that has no value), `v_head_dim` (values of another size than queries and keys), `names` (what the q, k, v,
    o matrices, the two norms and a bias are called under `prefix`)."""

    NAMES = ("q_proj.weight", "k_proj.weight", "v_proj.weight", "o_proj.weight", "q_norm.weight", "k_norm.weight", "{}.bias")

    def __init__(self, prefix: str, hidden: int, heads: int, kv_heads: int, head_dim: int, qk_norm: bool, norm_eps: float,
                 position: base.PositionEncoding, window: Optional[int] = None, own_kv: bool = True, scale: Optional[float] = None,
                 bias: bool = False, softcap: Optional[float] = None, sink: bool = False, v_head_dim: Optional[int] = None, names: tuple = NAMES):
        if heads % kv_heads:
            raise ValueError(f"{heads} query heads are not a multiple of {kv_heads} kv heads")
        if getattr(position, "pairing", "half") != "half":
            raise ValueError("this attention turns entry i with i + rotary_dim/2: it needs a position encoding with pairing=\"half\"")
        if softcap is not None and not softcap > 0:
            raise ValueError(f"softcap must be positive, got {softcap}")
        if bias and not own_kv:
            raise ValueError("an attention that reads another layer's cache has no biased k and v projections")
        self.prefix, self.hidden, self.heads, self.kv_heads, self.head_dim = prefix, hidden, heads, kv_heads, head_dim
        self.v_head_dim = v_head_dim or head_dim
        self.qk_norm, self.norm_eps, self.position, self.window, self.own_kv = qk_norm, norm_eps, position, window, own_kv
        self.scale = scale if scale is not None else 1.0 / math.sqrt(head_dim)  # crates/specrt/src/codegen.rs:147
        self.bias, self.softcap, self.sink, self.names = bool(bias), softcap, bool(sink), tuple(names)
        self.wqkv = self.wo = self.q_norm = self.k_norm = self.qkv_bias = None

    @property
    def plain(self) -> bool:
        """The form every attention kernel of the engine computes: one head size, no bias, plain scores, plain softmax."""
        return not (self.bias or self.softcap or self.sink) and self.v_head_dim == self.head_dim

    def cache_need(self):
        # one row size for keys and values: the larger of the two (the kernels are told both)
        return PagedKV(self.kv_heads, max(self.head_dim, self.v_head_dim), self.window) if self.own_kv else None

    def _n(self, i: int) -> str:
        return f"{self.prefix}.{self.names[i]}"

    def _b(self, i: int) -> str:
        """The bias of matrix i: its name without a trailing ".weight", in the bias pattern."""
        stem = self.names[i][:-len(".weight")] if self.names[i].endswith(".weight") else self.names[i]
        return f"{self.prefix}.{self.names[6].format(stem)}"

    def weight_specs(self):
        hd, vd = self.head_dim, self.v_head_dim
        sizes = [self.heads * hd, self.kv_heads * hd, self.kv_heads * vd]
        specs = [WeightSpec(self._n(0), (sizes[0], self.hidden)), WeightSpec(self._n(3), (self.hidden, self.heads * vd))]
        if self.own_kv:
            specs += [WeightSpec(self._n(1), (sizes[1], self.hidden)), WeightSpec(self._n(2), (sizes[2], self.hidden))]
        if self.qk_norm:
            specs.append(WeightSpec(self._n(4), (hd,), role="norm"))
            if self.own_kv:
                specs.append(WeightSpec(self._n(5), (hd,), role="norm"))
        if self.bias:
            specs += [WeightSpec(self._b(i), (sizes[i],), std=0.1) for i in range(3)] + [WeightSpec(self._b(3), (self.hidden,), std=0.1)]
        return specs

    def bind(self, weights, rt):
        rows = [weights[self._n(0)]]
        if self.own_kv:
            rows += [weights[self._n(1)], weights[self._n(2)]]
        else:  # keep the [q | k | v] row layout the kernels read; the k and v rows are never used
            z = torch.zeros((self.kv_heads * (self.head_dim + self.v_head_dim), self.hidden), dtype=rows[0].dtype, device=rows[0].device)
            rows.append(z)
        self.wqkv = rt.matrix(torch.cat(rows, dim=0))
        self.wo = rt.matrix(weights[self._n(3)])
        if self.qk_norm:
            self.q_norm = rt.vector(weights[self._n(4)])
            if self.own_kv:
                self.k_norm = rt.vector(weights[self._n(5)])
        if self.bias:
            self.qkv_bias = rt.vector(torch.cat([weights[self._b(i)].to(torch.float32) for i in range(3)]))
            self.out_bias = rt.vector(weights[self._b(3)])
        self.position.bind(weights, rt)

    adds_to_residual = True   # the output projection may add to the residual stream in its epilogue

    def _forward_variant(self, ctx, h, cache):
        """Any of the variants: the projection's partial sums go through the q/k kernel that adds biases and takes two head sizes, then
        the attention kernels that cap scores and count the sink."""
        rt = ctx.rt
        from ..kernels import attention
        cos, sin = self.position.tables(ctx)
        qkv = rt.linear(h, self.wqkv)
        q = rt.empty((ctx.n_tokens, self.heads * self.head_dim))
        ops.qk_norm_rope_kv(qkv, self.q_norm, self.k_norm, self.norm_eps, cos, sin, ctx.positions, ctx.seg_of_token, q, cache, self.heads,
                            rt.status, write_kv=self.own_kv, bias=self.qkv_bias, qk_dim=self.head_dim, v_dim=self.v_head_dim)
        out = attention.paged_attention(ctx, q, cache, self.heads, self.window, self.scale, qk_dim=self.head_dim, v_dim=self.v_head_dim,
                                        softcap=self.softcap or 0.0, sink=self.sink)
        return rt.linear(out, self.wo)

    def forward(self, ctx, h, cache, residual=None):
        rt = ctx.rt
        if not self.plain:
            return self._forward_variant(ctx, h, cache)
        cos, sin = self.position.tables(ctx)
        from ..kernels import attention
        q = attention.project_qkv(ctx, h, self.wqkv, self.q_norm, self.k_norm, self.norm_eps, cos, sin, cache, self.heads, self.own_kv)
        if q is not None:   # many tokens: norm, rotation and cache write happened in the projection's epilogue
            out = attention.paged_attention(ctx, q, cache, self.heads, self.window, self.scale)
            return rt.linear(out, self.wo, add_to=residual)
        qkv = rt.linear(h, self.wqkv)
        out = attention.decode_fused(ctx, qkv, self.q_norm, self.k_norm, self.norm_eps, cos, sin, cache, self.heads, self.window, self.scale, self.own_kv)
        if out is None:   # not a step of decoded tokens only, or sizes the fused kernel does not have
            q = rt.empty((ctx.n_tokens, self.heads * self.head_dim))
            ops.qk_norm_rope_kv(qkv, self.q_norm, self.k_norm, self.norm_eps, cos, sin, ctx.positions, ctx.seg_of_token, q, cache, self.heads,
                                rt.status, write_kv=self.own_kv)
            out = attention.paged_attention(ctx, q, cache, self.heads, self.window, self.scale)
        return rt.linear(out, self.wo, add_to=residual)


# ------------------------------------------------------------------------------------------ feed-forward
@base.register_feed_forward("swiglu")
class SwiGLU(base.FeedForward):
    """down(silu(gate h) * up h), silu(g) = g / (1 + exp(-g)) in float32
    (crates/kir/src/cuda/prelude.cu:125-133; gate and up fused into one product at load,
    crates/specrt/src/weights.rs:1049-1062)."""

    def __init__(self, prefix: str, hidden: int, intermediate: int, names: tuple = ("gate_proj.weight", "up_proj.weight", "down_proj.weight")):
        """names: what the gate, up and down matrices are called under `prefix`."""
        self.prefix, self.hidden, self.intermediate, self.names = prefix, hidden, intermediate, tuple(names)
        self.wgu = self.wd = None

    def weight_specs(self):
        p, (g, u, d) = self.prefix, self.names
        return [WeightSpec(f"{p}.{g}", (self.intermediate, self.hidden)), WeightSpec(f"{p}.{u}", (self.intermediate, self.hidden)),
                WeightSpec(f"{p}.{d}", (self.hidden, self.intermediate))]

    def bind(self, weights, rt):
        p, (g, u, d) = self.prefix, self.names
        self.wgu = rt.matrix(torch.cat([weights[f"{p}.{g}"], weights[f"{p}.{u}"]], dim=0))
        self.wd = rt.matrix(weights[f"{p}.{d}"])

    adds_to_residual = True   # the down projection may add to the residual stream in its epilogue

    def forward(self, ctx, h, residual=None):
        rt = ctx.rt
        return rt.linear(rt.gate_up_act(h, self.wgu), self.wd, add_to=residual)


@base.register_feed_forward("dense_xielu")
class DenseXielu(base.FeedForward):
    """down(act(up h)) with the activation xIELU, whose two numbers (p, q) are a tensor of the layer:
    act(z) = softplus(p) z^2 + z / 2 for z > 0, (1/2 + softplus(q)) (exp(z) - 1 - z) + z / 2 otherwise, in float32 on the product's
    float32 sums (`Runtime.up_xielu`: in the tensor-core product's epilogue where its k-range is whole)."""

    def __init__(self, prefix: str, hidden: int, intermediate: int, names: tuple = ("up", "down", "act")):
        self.prefix, self.hidden, self.intermediate, self.names = prefix, hidden, intermediate, tuple(names)
        self.wu = self.wd = self.pq = None

    def weight_specs(self):
        p, (u, d, a) = self.prefix, self.names
        return [WeightSpec(f"{p}.{u}", (self.intermediate, self.hidden)), WeightSpec(f"{p}.{d}", (self.hidden, self.intermediate)),
                WeightSpec(f"{p}.{a}", (2,), std=0.5)]

    def bind(self, weights, rt):
        p, (u, d, a) = self.prefix, self.names
        self.wu, self.wd, self.pq = rt.matrix(weights[f"{p}.{u}"]), rt.matrix(weights[f"{p}.{d}"]), rt.vector(weights[f"{p}.{a}"])

    adds_to_residual = True   # the down projection may add to the residual stream in its epilogue

    def forward(self, ctx, h, residual=None):
        rt = ctx.rt
        return rt.linear(rt.up_xielu(h, self.wu, self.pq), self.wd, add_to=residual)


# ------------------------------------------------------------------------------------------ embedding and head
@base.register_embedding("table")
class TokenEmbedding(base.Embedding):
    """x[t] = float32(E[token_t]) * 1 (crates/kir/src/prims.rs:387)."""

    def __init__(self, name: str, vocab: int, hidden: int, scale: float = 1.0, positions: Optional[str] = None, max_positions: int = 0):
        """scale: a constant on the token's vector. positions: the name of a table [max_positions, hidden] of learned vectors, one a position,
        added to it unscaled: x[t] = E[token_t] * scale + P[position_t]."""
        if positions is not None and max_positions <= 0:
            raise ValueError("a table of learned positions needs its number of positions")
        self.name, self.vocab, self.hidden, self.scale, self.positions, self.max_positions = name, vocab, hidden, float(scale), positions, max_positions
        self.table = self.pos_table = None

    def weight_specs(self):
        specs = [WeightSpec(self.name, (self.vocab, self.hidden))]
        if self.positions is not None:
            specs.append(WeightSpec(self.positions, (self.max_positions, self.hidden)))
        return specs

    def bind(self, weights, rt):
        self.table = rt.matrix(weights[self.name])
        if self.positions is not None:
            self.pos_table = rt.matrix(weights[self.positions])

    def forward(self, ctx):
        x = ctx.rt.empty((ctx.n_tokens, self.hidden), torch.float32)
        if self.pos_table is None and self.scale == 1.0:
            ops.embed(self.table.weight, ctx.token_ids, x, ctx.rt.status)
        elif self.pos_table is None:
            ops.embed(self.table.weight, ctx.token_ids, x, ctx.rt.status)
            ops.scale_values(x, self.scale)
        else:
            ops.embed_pos(self.table.weight, ctx.token_ids, self.pos_table.weight, ctx.positions, self.scale, x, ctx.rt.status)
        return x


@base.register_head("linear")
class LinearHead(base.Head):
    """logits = W h in float32; `tied_to` names the embedding table to use instead of a matrix of
    its own (a tied model ignores lm_head.weight even when the file has it:
    crates/specrt/src/weights.rs:1396-1405)."""

    def __init__(self, name: str, vocab: int, hidden: int, tied_to: Optional[str] = None, scale: float = 1.0):
        """scale: a constant on the logits."""
        self.name, self.vocab, self.hidden, self.tied_to, self.scale = name, vocab, hidden, tied_to, float(scale)
        self.w = None

    def weight_specs(self):
        return [WeightSpec(self.tied_to or self.name, (self.vocab, self.hidden))]   # tied: the embedding's table, read by both

    def bind(self, weights, rt):
        self.w = rt.matrix(weights[self.tied_to or self.name])

    def forward(self, ctx, h):
        out = ctx.rt.linear(h, self.w, allow_split=False)
        if out.shape[0] != 1:
            raise RuntimeError(f"the head's product came back in {out.shape[0]} partial sums although it asked for one")
        if self.scale != 1.0:
            ops.scale_values(out[0], self.scale)
        return out[0]


# ------------------------------------------------------------------------------------------ block
@base.register_block("prenorm")
class PreNormBlock(base.Block):
    """x += mixer(norm(x)); x += feed_forward(norm(x)) (crates/specrt/graphs/decoder.toml:168-303).
    Each residual add is fused into the norm that follows it, so the feed-forward's contribution
    is handed to the next block (or the final norm) instead of being added here."""

    def __init__(self, mixer_norm, mixer, feed_forward_norm, feed_forward):
        super().__init__(mixer_norm, mixer, feed_forward_norm, feed_forward)
        if getattr(mixer, "bias", False):
            raise ValueError("this arrangement does not add a mixer's output bias")

    def forward(self, ctx, x, pending, cache):
        h = self.mixer_norm.forward(ctx, x, pending)
        a = self.mixer.forward(ctx, h, cache, residual=x) if self.mixer.adds_to_residual else self.mixer.forward(ctx, h, cache)
        h = self.feed_forward_norm.forward(ctx, x, a)
        return self.feed_forward.forward(ctx, h, residual=x) if self.feed_forward.adds_to_residual else self.feed_forward.forward(ctx, h)


@base.register_block("outnorm")
class OutNormBlock(base.Block):
    """x += m * norm(mixer(x)); x += m * norm(feed_forward(x)): the sublayers read the residual stream itself and the norm
    sits on what they give back, scaled by a residual multiplier m. The stream stays float32; its rounding to the
    activation dtype, which the next sublayer reads, is written by the kernel that adds to it. A layer without a
    feed-forward (`feed_forward` of kind "none") has the first half only."""

    def __init__(self, mixer_norm, mixer, feed_forward_norm, feed_forward, residual_mult: float = 1.0):
        super().__init__(mixer_norm, mixer, feed_forward_norm, feed_forward)
        if getattr(mixer, "bias", False):
            raise ValueError("this arrangement does not add a mixer's output bias")
        self.residual_mult = residual_mult

    def forward(self, ctx, x, pending, cache):
        if pending is not None:
            raise RuntimeError("an outnorm block follows a block that left a contribution to add: mixing arrangements is not supported")
        key = ("outnorm act", x.data_ptr())
        h = ctx.memo.get(key)
        if h is None:   # the first block of a step: the embedding's rows
            h = x if ctx.rt.act_dtype == torch.float32 else ctx.rt.empty(tuple(x.shape))
            if h is not x:
                ops.cast_rows(x, h)
        a = self.mixer.forward(ctx, h, cache)
        h = self.mixer_norm.add_normed(ctx, x, a, self.residual_mult)
        if not isinstance(self.feed_forward, NoFeedForward):
            f = self.feed_forward.forward(ctx, h)
            h = self.feed_forward_norm.add_normed(ctx, x, f, self.residual_mult)
        ctx.memo[key] = h
        return None


@base.register_block("sandwich")
class SandwichBlock(base.Block):
    """x += post1(mixer(norm1(x))); x += post2(feed_forward(norm2(x))): a norm in front of every sublayer and another on what it gives back.
    The two output norms are the arrangement's own parts (`post_norms`: two `PartSpec`-built norms handed in by the plan as parameters).
    Each output norm runs in the kernel of the input norm that follows it: post1 with norm2, post2 with the next block's norm1 (or the final
    norm), to which the feed-forward's contribution goes as a `NormedDelta`. A mixer's output bias is added before post1. A layer without a
    feed-forward has the first half only."""

    takes_out_bias = True

    def __init__(self, mixer_norm, mixer, feed_forward_norm, feed_forward, post_mixer_norm=None, post_feed_forward_norm=None):
        base.Block.__init__(self, mixer_norm, mixer, feed_forward_norm, feed_forward)
        self.has_ff = not isinstance(feed_forward, NoFeedForward)
        norms = [mixer_norm, post_mixer_norm] + ([feed_forward_norm, post_feed_forward_norm] if self.has_ff else [])
        if any(not isinstance(n, RMSNorm) for n in norms) or len({n.eps for n in norms}) != 1:
            raise ValueError("this arrangement is built for four RMS norms with one epsilon")
        self.post_mixer_norm, self.post_feed_forward_norm = post_mixer_norm, post_feed_forward_norm

    def parts(self):
        return [*base.Block.parts(self), self.post_mixer_norm] + ([self.post_feed_forward_norm] if self.has_ff else [])

    def forward(self, ctx, x, pending, cache):
        if pending is not None and not isinstance(pending, base.NormedDelta):
            raise RuntimeError("this block follows a block that left a plain contribution to add: mixing arrangements is not supported")
        h = self.mixer_norm.forward(ctx, x, pending)
        a = self.mixer.forward(ctx, h, cache)
        if not self.has_ff:
            return base.NormedDelta(a, self.post_mixer_norm, self.mixer.out_bias)
        h = self.post_mixer_norm.add_post(ctx, x, a, self.mixer.out_bias, self.feed_forward_norm)
        return base.NormedDelta(self.feed_forward.forward(ctx, h), self.post_feed_forward_norm)


@base.register_feed_forward("none")
class NoFeedForward(base.FeedForward):
    """A layer that has a mixer only."""

    def __init__(self):
        pass

    def forward(self, ctx, h):
        raise RuntimeError("a layer without a feed-forward has nothing to run")


@base.register_norm("none")
class NoNorm(base.Norm):
    """The place of a norm in a layer that has nothing to norm there."""

    def __init__(self):
        pass
