"""Gated feed-forward: down(act(gate(x), up(x))).

"gated_silu" (SwiGLU): act(g, u) = silu(g) * u.  "gated_relu": act(g, u) =
max(g, 0) * u.  "gated_clamped": with a limit
L and a slope a, g' = min(g, L), u' = clamp(u, -L, L), act = g' * sigmoid(a g')
* (u' + 1).

Gate and up are one projection [2 I, H], gate rows first, as the reference
fuses them at load (python/lyapunov_engine/models/weight_loader.py:155-163;
python/lyapunov_engine/models/llama.py:109-122).  The activation is computed in
32 bits and rounded once (csrc/kernels/fused_rmsnorm_swiglu.cu:170-176).
"""
from __future__ import annotations

import torch

from .. import ops
from .base import FeedForward, TensorDecl, register_feed_forward


@register_feed_forward("gated_silu")
class GatedFeedForward(FeedForward):
    activation = (ops.GLU_SILU, 1.0, 0.0)      # (kind, slope, limit) as the kernels take them

    def __init__(self, hidden_size: int, intermediate_size: int, gate_name: str, up_name: str, down_name: str):
        self.hidden_size, self.intermediate_size = int(hidden_size), int(intermediate_size)
        self.names = (gate_name, up_name, down_name)
        self.w_gate_up = self.w_down = None
        self.runtime = None

    def tensors(self):
        g, u, d = self.names
        H, I = self.hidden_size, self.intermediate_size
        return [TensorDecl(g, (I, H)), TensorDecl(u, (I, H)), TensorDecl(d, (H, I))]

    def bind(self, get, runtime):
        g, u, d = self.names
        self.w_gate_up = torch.cat([get(g), get(u)], dim=0).contiguous()
        self.w_down = get(d)
        self.runtime = runtime

    def forward(self, x, ctx):
        rt = self.runtime
        T = x.shape[0]
        ws = ctx.workspace
        act = ws.get("ffn_act", (T, self.intermediate_size), rt.dtype)
        ops.gated_linear(act, x, self.w_gate_up, ws, ctx.status, self.activation)
        return ops.linear_for_residual(act, self.w_down, ws, "ffn_out", ctx.status)

    def forward_plain(self, x, ctx, key: str = "ffn_plain"):
        """The same as one tensor [T, H] in the activations' type (``forward``
        may return partial sums for the norm to add), for a caller that goes
        on computing with it; buffers of its own, so that it can run inside
        another feed-forward."""
        rt = self.runtime
        ws = ctx.workspace
        act = ws.get(key + "_act", (x.shape[0], self.intermediate_size), rt.dtype)
        ops.gated_linear(act, x, self.w_gate_up, ws, ctx.status, self.activation)
        out = ws.get(key, (x.shape[0], self.hidden_size), rt.dtype)
        ops.linear(out, act, self.w_down, ctx.status)
        return out


@register_feed_forward("gated_relu")
class ReluGatedFeedForward(GatedFeedForward):
    activation = (ops.GLU_RELU, 1.0, 0.0)


@register_feed_forward("gated_clamped")
class ClampedGatedFeedForward(GatedFeedForward):
    def __init__(self, hidden_size: int, intermediate_size: int, gate_name: str, up_name: str, down_name: str,
                 limit: float, slope: float = 1.702):
        super().__init__(hidden_size, intermediate_size, gate_name, up_name, down_name)
        if not limit > 0:
            raise ValueError(f"the clamped activation needs a positive limit, got {limit}")
        self.activation = (ops.GLU_CLAMPED, float(slope), float(limit))
