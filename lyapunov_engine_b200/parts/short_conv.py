"""A short causal convolution over time, added to its own input:

    y[t] = x[t] + sum_{j < taps} w[:, j] * x[t - (taps - 1 - j)]      (per channel)

with x before a request's start taken as zero.  A block may put it between a
norm and the sub-layer that reads the norm's output.  The last ``taps - 1``
inputs of every request are per-request state (one row per state slot), so a
request continues exactly where its last step ended, however its tokens are
cut into steps.  The weight is stored [channels, taps] and kept transposed,
32-bit.
"""
from __future__ import annotations

import torch

from .. import ops
from .base import InputFilter, StateNeed, TensorDecl, register_input_filter


@register_input_filter("causal_taps")
class CausalTaps(InputFilter):
    def __init__(self, channels: int, taps: int, weight_name: str):
        self.channels, self.taps, self.weight_name = int(channels), int(taps), weight_name
        if not 1 <= self.taps <= ops.SHORT_CONV_MAX_TAPS:
            raise ValueError(f"a short convolution takes 1..{ops.SHORT_CONV_MAX_TAPS} taps, got {taps}")
        self.weight = None
        self.runtime = None

    def state_need(self):
        if self.taps == 1:
            return None
        return StateNeed((self.taps - 1, self.channels), torch.float32)

    def tile_sizes(self):
        return [ops.SHORT_CONV_TILE]

    def tensors(self):
        return [TensorDecl(self.weight_name, (self.channels, self.taps), role="vector", init="taps")]

    def bind(self, get, runtime):
        self.weight = get(self.weight_name).t().contiguous()        # [taps, channels]
        self.runtime = runtime

    def forward(self, x, ctx, state):
        out = ctx.workspace.get("filtered", tuple(x.shape), x.dtype)
        if ctx.pure_decode:
            # one token per request: request b is row b, no tile list to read
            ops.short_conv(out, x, self.weight, state, ctx.state_slots, ctx.cu_q, None, None, ctx.num_requests)
        else:
            tile_request, tile_q0, num_tiles, _ = ctx.tiles[ops.SHORT_CONV_TILE]
            ops.short_conv(out, x, self.weight, state, ctx.state_slots, ctx.cu_q, tile_request, tile_q0, num_tiles)
        return out
