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

import os

import torch

from .. import ops
from .base import InputFilter, StateNeed, TensorDecl, register_input_filter


# 0: the norm before the filter and the filter always run as two kernels
FUSE_WITH_NORM = os.environ.get("LYAPUNOV_FUSE_TAPS", "1") not in ("0", "")


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

    def after_norm(self, norm, resid, delta, ctx, state):
        """The norm before this filter and the filter as one kernel, where that
        exists: steps whose requests all bring one token, an RMS norm (whole
        or in groups) over rows the kernel holds in registers.  None: nothing
        was done, the caller runs the norm and forward()."""
        if not (FUSE_WITH_NORM and ctx.pure_decode and ctx.num_tokens == ctx.num_requests):
            return None
        if getattr(norm, "weight", None) is None or not hasattr(norm, "groups") or norm.hidden_size != self.channels:
            return None
        if not ops.rmsnorm_taps_applies(self.channels, norm.groups):
            return None
        out = ctx.workspace.get("filtered", (ctx.num_tokens, self.channels), self.runtime.dtype)
        ops.rmsnorm_taps(out, resid, delta, norm.weight, norm.eps, norm.groups, self.weight, state, ctx.state_slots)
        return out

    def forward(self, x, ctx, state):
        out = ctx.workspace.get("filtered", tuple(x.shape), x.dtype)
        if ctx.pure_decode:
            # one token per request: request b is row b, no tile list to read
            ops.short_conv(out, x, self.weight, state, ctx.state_slots, ctx.cu_q, None, None, ctx.num_requests)
        else:
            tile_request, tile_q0, num_tiles, _ = ctx.tiles[ops.SHORT_CONV_TILE]
            ops.short_conv(out, x, self.weight, state, ctx.state_slots, ctx.cu_q, tile_request, tile_q0, num_tiles)
        return out
