"""Differential attention over the paged cache.

Every query head carries ``maps`` (two) attention maps: its projection rows are
[map 1 | map 2], ``head_dim`` each, and so are the rows of its key head; both
maps attend over the same values.  With a_m the maps' outputs,
    o = a_1 - lam * a_2,   lam = exp(lq1 . lk1) - exp(lq2 . lk2) + diff
(one number per layer from four learned vectors and the constant ``diff``),
then o / sqrt(mean(o^2) + eps) over the head's values, times (1 - diff), then
the output projection.  Queries, keys and values may have biases.  Positions:
rotary on the first ``rot`` entries of every map, neighbouring entries paired.
Keys are visible through a sliding window or all.

How it runs on the kernels that serve grouped-query attention: a key head in
the cache is the kv head's maps side by side (maps * head_dim wide, the size
the projection gives it); each (query head, map) becomes a query head of that
width with its map's columns filled and zeros elsewhere, so its dot product
with the whole key is its own map's score, and maps * heads query heads share
kv_heads key/value heads.  The cache holds every key and value once; the price
is a score product of maps times the needed width.  One kernel adds the
biases, rotates, spreads the queries and writes the cache; one combines the
maps' outputs (see ops.rope_pairs_store, ops.maps_combine).
"""
from __future__ import annotations

import math

import torch

from .. import ops
from . import attention_kernels
from .base import KVNeed, Mixer, TensorDecl, register_mixer


@register_mixer("differential_attention")
class DifferentialAttentionMixer(Mixer):
    def __init__(self, hidden_size: int, num_heads: int, num_kv_heads: int, head_dim: int, value_dim: int, scale: float,
                 diff: float, norm_eps: float, rot: int, rot_base: float, q_name: str, k_name: str, v_name: str, o_name: str,
                 lambda_names: tuple, window: int | None = None, maps: int = 2, bias_names: tuple | None = None):
        if num_heads % num_kv_heads:
            raise ValueError(f"{num_heads} heads do not divide into {num_kv_heads} groups")
        if maps != 2 or len(lambda_names) != 4:
            raise ValueError("differential attention has two maps per head and four lambda vectors")
        self.hidden_size, self.num_heads, self.num_kv_heads = int(hidden_size), int(num_heads), int(num_kv_heads)
        self.maps, self.map_dim, self.value_dim = int(maps), int(head_dim), int(value_dim)
        # the one head size of kernels and pages
        self.head_dim = (max(self.maps * self.map_dim, self.value_dim) + 15) // 16 * 16
        if not 16 <= self.head_dim <= attention_kernels.MAX_HEAD_DIM:
            raise ValueError(f"attention takes head sizes up to {attention_kernels.MAX_HEAD_DIM}; {maps} maps of {head_dim} "
                             f"and values of {value_dim} need {self.head_dim}")
        self.rot = int(rot)
        if self.rot % 2 or not 0 <= self.rot <= self.map_dim:
            raise ValueError(f"rotary width {rot} must be even and at most the map size {head_dim}")
        self.rot_base = float(rot_base)
        self.scale, self.diff, self.norm_eps = float(scale), float(diff), float(norm_eps)
        self.window = int(window) if window else None
        self.reach = ops.reach_code(self.window, None)
        self.names = (q_name, k_name, v_name, o_name)
        self.lambda_names = tuple(lambda_names)
        self.bias_names = tuple(bias_names) if bias_names else None
        self.w_qkv = self.w_o = self.bias = self.rates = self.coef = None
        self.runtime = None

    @property
    def query_heads(self) -> int:
        return self.num_heads * self.maps

    def cache_need(self):
        return KVNeed(self.num_kv_heads, self.head_dim, self.window, None)

    def tile_sizes(self):
        return attention_kernels.tile_sizes()

    def decode_variant(self, fill, num_decode, context_bound):
        if self.runtime is None or self.runtime.dtype != torch.bfloat16:
            return None
        return attention_kernels.decode_variant(fill, self.query_heads, self.num_kv_heads, self.head_dim, context_bound,
                                                self.reach)

    def tensors(self):
        q, k, v, o = self.names
        W, H, G, d, e, m = self.hidden_size, self.num_heads, self.num_kv_heads, self.map_dim, self.value_dim, self.maps
        decls = [TensorDecl(q, (H * m * d, W)), TensorDecl(k, (G * m * d, W)), TensorDecl(v, (G * e, W)),
                 TensorDecl(o, (W, H * e))]
        if self.bias_names:
            bq, bk, bv = self.bias_names
            decls += [TensorDecl(bq, (H * m * d,), role="vector", init="zeros"),
                      TensorDecl(bk, (G * m * d,), role="vector", init="zeros"),
                      TensorDecl(bv, (G * e,), role="vector", init="zeros")]
        decls += [TensorDecl(n, (d,), role="vector", init="zeros") for n in self.lambda_names]
        return decls

    def bind(self, get, runtime):
        q, k, v, o = self.names
        self.w_qkv = torch.cat([get(q), get(k), get(v)], dim=0).contiguous()
        self.w_o = get(o)
        self.bias = torch.cat([get(n) for n in self.bias_names]).contiguous() if self.bias_names else None
        i = torch.arange(0, self.rot, 2, dtype=torch.float64)
        rates = torch.pow(torch.tensor(self.rot_base, dtype=torch.float64), -i / max(self.rot, 1))
        self.rates = rates.to(torch.float32).to(runtime.device).contiguous()
        lq1, lk1, lq2, lk2 = (get(n).double().cpu() for n in self.lambda_names)
        lam = math.exp(float((lq1 * lk1).sum())) - math.exp(float((lq2 * lk2).sum())) + self.diff
        self.lam = lam
        self.coef = torch.tensor([1.0, -lam], dtype=torch.float32, device=runtime.device)
        self.runtime = runtime
        attention_kernels.prepare(self.head_dim)

    def forward(self, x, ctx, cache):
        rt = self.runtime
        H, G, hd = self.num_heads, self.num_kv_heads, self.head_dim
        T = x.shape[0]
        ws = ctx.workspace
        kv = cache.kv
        qkv = ws.get("qkv", (T, self.w_qkv.shape[0]), rt.dtype)
        ops.linear(qkv, x, self.w_qkv, ctx.status)
        q_wide = ws.get("q_maps", (T, self.query_heads * hd), rt.dtype)
        ops.rope_pairs_store(q_wide, qkv, self.bias, kv.k, kv.v, self.rates, ctx.positions, ctx.request_of_token,
                             ctx.block_tables[kv.group], H, G, self.maps, self.map_dim, self.value_dim, self.rot, hd,
                             kv.page_size, cache.write, ctx.status)
        attn = ws.get("attn", (T, self.query_heads * hd), rt.dtype)
        attention_kernels.run(attn, q_wide, ctx, kv, self.query_heads, G, hd, self.reach, self.scale)
        o = ws.get("attn_heads", (T, H * self.value_dim), rt.dtype)
        ops.maps_combine(o, attn, self.coef, H, self.maps, hd, self.value_dim, self.norm_eps, 1.0 - self.diff)
        return ops.linear_for_residual(o, self.w_o, ws, "mixer_out", ctx.status)
