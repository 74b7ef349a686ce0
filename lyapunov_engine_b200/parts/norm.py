"""Norms over the 32-bit residual stream (with the residual addition fused):
RMSNorm, and LayerNorm with weight and bias, which also reads a stream kept
in several copies.

Reference: rmsnorm (python/lyapunov_engine/ops.py:12-51) and rmsnorm_kernel
(csrc/kernels/fused_rmsnorm_swiglu.cu:15-113); the layer's norm weights there
are bare parameters of the decoder layer (python/lyapunov_engine/models/llama.py:130-134).
"""
from __future__ import annotations

from .. import ops
from .base import Norm, TensorDecl, register_norm


@register_norm("rmsnorm")
class RMSNorm(Norm):
    """``groups`` > 1: the row is cut into that many equal consecutive parts,
    each divided by its own sqrt(mean(part^2) + eps), before the weight."""

    def __init__(self, hidden_size: int, eps: float, weight_name: str, groups: int = 1):
        self.hidden_size = int(hidden_size)
        self.groups = int(groups)
        if self.groups < 1 or self.hidden_size % self.groups:
            raise ValueError(f"a norm over {hidden_size} values cannot be cut into {groups} equal parts")
        self.eps = float(eps)
        self.weight_name = weight_name
        self.weight = None
        self.runtime = None

    def tensors(self):
        return [TensorDecl(self.weight_name, (self.hidden_size,), role="vector", init="ones_jitter")]

    def bind(self, get, runtime):
        self.weight = get(self.weight_name)
        self.runtime = runtime

    def apply(self, resid, delta=None, rows=None, workspace=None, key="normed"):
        n = resid.shape[0] if rows is None else rows.shape[0]
        ws = workspace or self.runtime.workspace
        out = ws.get(key, (n, self.hidden_size), self.runtime.dtype)
        ops.rmsnorm(out, resid, delta, self.weight, self.eps, rows, groups=self.groups)
        return out


@register_norm("layernorm")
class LayerNorm(Norm):
    """(x - mean) / sqrt(var + eps) * w + b with var the mean of the squared
    deviations, in 32 bits.  It reads a residual stream in one copy or in
    several (see ``apply_stream``): the pending update of the copies, the
    reading sub-layer's weighted sum of them and the norm are one kernel."""

    def __init__(self, hidden_size: int, eps: float, weight_name: str, bias_name: str):
        self.hidden_size = int(hidden_size)
        self.eps = float(eps)
        self.weight_name, self.bias_name = weight_name, bias_name
        self.weight = self.bias = None
        self.runtime = None

    def tensors(self):
        return [TensorDecl(self.weight_name, (self.hidden_size,), role="vector", init="ones_jitter"),
                TensorDecl(self.bias_name, (self.hidden_size,), role="vector", init="zeros")]

    def bind(self, get, runtime):
        self.weight, self.bias = get(self.weight_name), get(self.bias_name)
        self.runtime = runtime

    def _out(self, n, workspace, key):
        ws = workspace or self.runtime.workspace
        return ws.get(key, (n, self.hidden_size), self.runtime.dtype)

    def apply(self, resid, delta=None, rows=None, workspace=None, key="normed"):
        out = self._out(resid.shape[0] if rows is None else rows.shape[0], workspace, key)
        ops.stream_norm(out, resid.view(resid.shape[0], 1, self.hidden_size), self.weight, self.bias, self.eps, delta=delta,
                        rows=rows)
        return out

    def apply_stream(self, stream, read=None, rows=None, workspace=None, key="normed"):
        T, W = stream.resid.shape[0], self.hidden_size
        copies = read.copies if read is not None else stream.copies
        init = None
        if stream.copies != copies:
            # the first sub-layer that keeps several copies: each starts as the one there is
            if stream.copies != 1 or stream.pending is not None or rows is not None:
                raise ValueError(f"a stream in {stream.copies} copies cannot be read as {copies}")
            init = stream.resid
            ws = workspace or self.runtime.workspace
            stream.resid = ws.get("stream_copies", (T, copies, W), init.dtype)
            stream.copies = copies
        out = self._out(T if rows is None else rows.shape[0], workspace, key)
        update = stream.update
        ops.stream_norm(out, stream.resid.view(T, copies, W), self.weight, self.bias, self.eps, delta=stream.pending,
                        mix=update.mix if update is not None else None, post=update.post if update is not None else None,
                        pre=read.pre if read is not None else None, init=init, rows=rows)
        if rows is None:
            stream.pending = stream.update = None
        return out
