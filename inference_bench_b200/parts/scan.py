"""A selective state-space scan as a mixer (the Mamba form).

With h the layer's input, per token:
    [u | z] = W_in h                                   (u, z of size `inner`)
    x = silu(conv(u) + b_conv)                          (a causal convolution per channel over `taps` tokens; zeros before the start)
    [dt_low | B | C] = W_x x                            (dt_low of size dt_rank; B, C of size `state`)
    dt = softplus(W_dt dt_low + b_dt);   A = -exp(A_log)
    S[c, n] <- exp(dt_c A[c, n]) S[c, n] + dt_c x_c B_n;   y_c = sum_n S[c, n] C_n + D_c x_c;   out = W_o (y * silu(z))
S [inner, state] is float32 state of the request (zero at admission), and so are the convolution's last taps - 1 inputs: two fixed-size
slots per request. Float32 whatever the activation dtype: the convolution's sum, x as the scan reads it, dt_low, B, C (taken from the
float32 sums of the product), the small product W_dt dt_low, softplus, the exponentials, the state and y. The matrix products W_in,
W_x and W_o read their inputs in the activation dtype.

Kernels: csrc/selective_scan.cu (`conv_silu`, `selective_scan`; the scan also writes the new convolution state, after every reader of
the old one). A segment of more than `ops.RECURRENCE_CHUNK` tokens is cut into chunks that are walked side by side: the decays of a
chunk multiply to exp(A * sum of its step sizes), so each chunk is walked from a zero state, the states are carried from chunk to
chunk, and each chunk is walked again from its incoming state for the outputs.
"""
from __future__ import annotations

import torch

from ..kernels import ops
from . import base
from .base import FixedState, Several, WeightSpec
from .recurrent import GatedLinearRecurrence


@base.register_mixer("mamba1")
class SelectiveScan(base.Mixer):
    def __init__(self, prefix: str, hidden: int, inner: int, state: int, dt_rank: int, taps: int,
                 names: tuple = ("in", "conv", "conv.b", "x", "dt", "dt.b", "A_log", "D", "o")):
        if min(hidden, inner, state, dt_rank, taps) <= 0:
            raise ValueError(f"inner {inner}, state {state}, dt_rank {dt_rank} and taps {taps} must be positive")
        if state > 256:
            raise ValueError(f"{state} states a channel are above the 256 the scan kernel holds")
        self.prefix, self.hidden, self.inner, self.state, self.dt_rank, self.taps, self.names = prefix, hidden, inner, state, dt_rank, taps, tuple(names)
        self.w_in = self.w_x = self.w_o = self.conv_w = self.conv_b = self.w_dt = self.dt_b = self.A = self.D = None

    def cache_need(self):
        return Several((FixedState((self.inner, self.state), torch.float32), FixedState((max(self.taps - 1, 1), self.inner), torch.float32)))

    def _n(self, i: int) -> str:
        return f"{self.prefix}.{self.names[i]}"

    def weight_specs(self):
        I, N, R = self.inner, self.state, self.dt_rank
        return [WeightSpec(self._n(0), (2 * I, self.hidden)), WeightSpec(self._n(1), (I, self.taps), std=0.3), WeightSpec(self._n(2), (I,), std=0.1),
                WeightSpec(self._n(3), (R + 2 * N, I)), WeightSpec(self._n(4), (I, R), std=0.2), WeightSpec(self._n(5), (I,), std=0.5),
                WeightSpec(self._n(6), (I, N), role="log_rate"), WeightSpec(self._n(7), (I,), role="norm"), WeightSpec(self._n(8), (self.hidden, I))]

    def bind(self, weights, rt):
        self.w_in, self.w_x, self.w_o = rt.matrix(weights[self._n(0)]), rt.matrix(weights[self._n(3)]), rt.matrix(weights[self._n(8)])
        # the taps are stored [channel, tap]; the kernel reads a tap's weights for neighbouring channels together: [tap, channel]
        self.conv_w, self.conv_b = rt.vector(weights[self._n(1)].t()), rt.vector(weights[self._n(2)])
        self.w_dt, self.dt_b, self.D = rt.vector(weights[self._n(4)]), rt.vector(weights[self._n(5)]), rt.vector(weights[self._n(7)])
        self.A = -torch.exp(rt.vector(weights[self._n(6)]))   # float32, once at load

    def forward(self, ctx, h, cache):
        rt, T = ctx.rt, ctx.n_tokens
        state, conv_state = cache[0].tensor, cache[1].tensor
        proj = rt.linear(h, self.w_in)                                          # [P, T, 2 inner] = [u | z]
        xc = rt.empty((T, self.inner), torch.float32)
        xa = xc if rt.act_dtype == torch.float32 else rt.empty((T, self.inner))
        ops.conv_silu(proj, self.conv_w, self.conv_b, conv_state, ctx.seg_of_token, ctx.seg_start, ctx.seg_slot, xc, None if xa is xc else xa)
        low = rt.linear(xa, self.w_x)                                           # [P, T, dt_rank + 2 state]
        y = rt.empty((T, self.inner))
        short, long_segs, chunks = GatedLinearRecurrence._cut(ctx)            # one table of long segments and their chunks for all recurrences of a step
        ops.selective_scan(xc, low, proj, self.w_dt, self.dt_b, self.A, self.D, state, conv_state, self.taps, ctx.seg_start, ctx.seg_slot, ctx.n_segments, y,
                           seg_list=short, long_segs=long_segs, chunks=chunks)
        return rt.linear(y, self.w_o)
