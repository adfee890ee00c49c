"""The entry of a pass over looped layers: layers that run several times in a row with the same weights (each pass with a cache or state
of its own: the plan's schedule names a layer once per pass) take their stream from the stream so far and the embedding's output:

    x <- W [x ; x0] + step[t]          (W [H, 2H] with x's columns first; step [passes, H]; t the number of the pass, from 0)

right before the first layer of every pass, the first included. The stream so far (with the contribution the layer before left) and x0
are packed side by side in the activation dtype, as the matrix product's input; x is reset to step[t] and the product is left for the
next norm to add, so the pass costs one row-wise kernel and one product.
"""
from __future__ import annotations

import torch

from ..kernels import ops
from . import base
from .base import WeightSpec


@base.register_stream_part("loop_entry")
class LoopEntry(base.StreamPart):
    needs_embedding = True

    def __init__(self, hidden: int, passes: int, names: tuple = ("loop.in", "loop.step")):
        if passes <= 0:
            raise ValueError(f"a loop needs at least one pass, got {passes}")
        self.hidden, self.passes, self.names = hidden, passes, tuple(names)
        self.w = self.steps = None

    def weight_specs(self):
        return [WeightSpec(self.names[0], (self.hidden, 2 * self.hidden)), WeightSpec(self.names[1], (self.passes, self.hidden), std=0.1)]

    def bind(self, weights, rt):
        self.w, self.steps = rt.matrix(weights[self.names[0]]), rt.vector(weights[self.names[1]])

    def forward(self, ctx, x, pending, x0, occurrence):
        rt = ctx.rt
        packed = rt.empty((ctx.n_tokens, 2 * self.hidden))
        ops.loop_pack(x, pending, x0, self.steps[occurrence], packed)
        return rt.linear(packed, self.w)
