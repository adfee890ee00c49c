"""A pre-norm block whose mixer reads its input through a token shift:

    h = norm1(x);   h_t <- h_t + (h_(t-1) - h_t) * shift   (per channel, with h as it was before the replacement; zeros before a
                                                            request's first token);   x <- x + mixer(h) + the mixer's output bias
    x <- x + feed_forward(norm2(x))                         (a layer may have no feed-forward)

The last normed row of a request is state (a fixed-size float32 slot per request and execution, beside the mixer's own cache or state).
Norm and shift are float32; the shifted row is rounded to the activation dtype once, as the input of the mixer's matrix product.

Kernels (csrc/token_shift.cu): a step whose requests all bring one token runs the residual add, the norm and the shift as one kernel
(`add_rmsnorm_ext` with the shift); otherwise the norm writes float32 rows and `token_shift_rows` shifts them, reads the old state and
writes the new one. A mixer's output bias is added by the norm that adds the mixer's contribution.
"""
from __future__ import annotations

import torch

from ..kernels import ops
from . import base
from .base import FixedState, Several, WeightSpec
from .standard import NoFeedForward


@base.register_block("prenorm_shift")
class PreNormShiftBlock(base.Block, base.Part):
    takes_out_bias = True

    def __init__(self, mixer_norm, mixer, feed_forward_norm, feed_forward, prefix: str, hidden: int, names: tuple = ("shift",)):
        base.Block.__init__(self, mixer_norm, mixer, feed_forward_norm, feed_forward)
        self.has_ff = not isinstance(feed_forward, NoFeedForward)
        for norm in (mixer_norm, feed_forward_norm) if self.has_ff else (mixer_norm,):
            if not hasattr(norm, "w") or not hasattr(norm, "eps") or getattr(norm, "unit_offset", None) is None:
                raise ValueError(f"this arrangement runs RMS norms in its own kernels; {type(norm).__name__} is not one")
        self.prefix, self.hidden, self.names = prefix, hidden, tuple(names)
        self.mix = None
        need = self.mixer.cache_need()
        self._mixer_needs = need.needs if isinstance(need, Several) else (need,)
        self._mixer_several = isinstance(need, Several)

    # ------------------------------------------------------------ as a part: its own tensor and state
    def parts(self):
        return [self, *base.Block.parts(self)]

    def weight_specs(self):
        return [WeightSpec(f"{self.prefix}.{self.names[0]}", (self.hidden,), role="unit")]

    def bind(self, weights, rt):
        self.mix = rt.vector(weights[f"{self.prefix}.{self.names[0]}"])

    def cache_need(self):
        return Several((*self._mixer_needs, FixedState((self.hidden,), torch.float32)))

    # ------------------------------------------------------------ one step
    def forward(self, ctx, x, pending, cache):
        rt = ctx.rt
        own = cache[-1].tensor
        mixer_cache = tuple(cache[:-1]) if self._mixer_several else cache[0]
        norm = self.mixer_norm
        h = rt.empty((ctx.n_tokens, self.hidden))
        if ctx.fixed_shape or ctx.n_segments == ctx.n_tokens:
            ops.add_rmsnorm_ext(x, pending, norm.w, norm.eps, h, shift=(self.mix, own, ctx.seg_slot))
        else:
            normed = rt.empty((ctx.n_tokens, self.hidden), torch.float32)
            ops.add_rmsnorm(x, pending, norm.w, normed, norm.eps)
            ops.token_shift_rows(normed, self.mix, own, ctx.seg_of_token, ctx.seg_start, ctx.seg_slot, h)
        a = self.mixer.forward(ctx, h, mixer_cache)
        bias = self.mixer.out_bias
        if not self.has_ff:
            if bias is not None:
                ops.add_bias_rows(a[0], bias)   # nothing of this block adds the contribution: the bias goes into its first partial sum
            return a
        norm = self.feed_forward_norm
        h = rt.empty((ctx.n_tokens, self.hidden))
        if bias is not None:
            ops.add_rmsnorm_ext(x, a, norm.w, norm.eps, h, bias=bias)
        else:
            ops.add_rmsnorm(x, a, norm.w, h, norm.eps)
        return self.feed_forward.forward(ctx, h, residual=x) if self.feed_forward.adds_to_residual else self.feed_forward.forward(ctx, h)
