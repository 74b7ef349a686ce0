"""Plain, slow, whole-sequence implementation of the Sulepel decoder.

The yardstick of the Sulepel tests: no cache, no batching, no kernels, one
function per mechanism, plain torch on the CPU.  It shares no code with the
product package.  Notation: W width, T tokens, H query heads, G key/value
heads, d query/key size, e value size, r latent size.

``round_to`` (a torch dtype or None) is where the serving pipeline rounds
activations between matrix products; None keeps everything in ``dtype``.
"""
from __future__ import annotations

import math

import torch


def _r(x, round_to):
    return x if round_to is None else x.to(round_to).to(x.dtype)


# --------------------------------------------------------------------------
# mechanisms
# --------------------------------------------------------------------------
def sinusoid(positions: torch.Tensor, width: int, dtype=torch.float32) -> torch.Tensor:
    """[T, W]: column 2i holds sin(p * 10000^(-2i/W)), column 2i+1 its cosine."""
    i = torch.arange(0, width, 2, dtype=torch.float64)
    rate = torch.pow(torch.tensor(10000.0, dtype=torch.float64), -i / width).to(dtype)
    angle = positions.to(dtype)[:, None] * rate[None, :]
    out = torch.zeros(positions.shape[0], width, dtype=dtype)
    out[:, 0::2] = angle.sin()[:, : (width + 1) // 2]
    out[:, 1::2] = angle.cos()[:, : width // 2]
    return out


def grouped_rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float, groups: int) -> torch.Tensor:
    """Each of ``groups`` consecutive equal parts of a row is divided by its own
    sqrt(mean(part^2) + eps); the whole row is then multiplied by the weight."""
    T, W = x.shape
    parts = x.view(T, groups, W // groups)
    parts = parts / torch.sqrt(parts.pow(2).mean(-1, keepdim=True) + eps)
    return parts.reshape(T, W) * weight


def causal_taps(h: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """h + conv(h): conv(h)[t] = sum_j w[:, j] * h[t - taps + 1 + j], with zeros
    before the sequence's start.  w: [W, taps]."""
    T, W = h.shape
    taps = w.shape[1]
    padded = torch.cat([torch.zeros(taps - 1, W, dtype=h.dtype), h], dim=0)
    out = h.clone()
    for j in range(taps):
        out = out + w[:, j] * padded[j:j + T]
    return out


def masked_softmax_attention(q, k, v, scale, visible) -> torch.Tensor:
    """q: [H, T, d], k: [H, T, d], v: [H, T, e]; scale: number or [H] tensor;
    visible: [T, T] bool (row: query, column: key).  Returns [H, T, e]."""
    s = torch.einsum("htd,hsd->hts", q, k)
    if torch.is_tensor(scale):
        s = s * scale.view(-1, 1, 1)
    else:
        s = s * scale
    s = s.masked_fill(~visible, float("-inf"))
    p = torch.softmax(s, dim=-1)
    return torch.einsum("hts,hse->hte", p, v)


def causal_mask(T: int) -> torch.Tensor:
    i = torch.arange(T)
    return i[None, :] <= i[:, None]


def chunk_mask(T: int, size: int) -> torch.Tensor:
    """Query i sees key j <= i of its own chunk: floor(i / size) == floor(j / size)."""
    i = torch.arange(T)
    return (i[None, :] <= i[:, None]) & ((i[None, :] // size) == (i[:, None] // size))


def latent_attention(h, w, p, cfg, eps, round_to=None) -> torch.Tensor:
    """Keys and values of every head are linear maps of one normed latent
    vector per token; no positions; causal; sigmoid gate per head."""
    T = h.shape[0]
    H, d, e, r = cfg["heads"], cfg["dim"], cfg["vdim"], cfg["kv_rank"]
    q = _r(h @ w[p + "q"].T, round_to)
    latent = _r(h @ w[p + "dkv"].T, round_to)
    latent = latent / torch.sqrt(latent.pow(2).mean(-1, keepdim=True) + eps) * w[p + "dkv.norm"]
    latent = _r(latent, round_to)
    k = _r(latent @ w[p + "uk"].T, round_to)
    v = _r(latent @ w[p + "uv"].T, round_to)
    assert k.shape[1] == H * d and v.shape[1] == H * e and latent.shape[1] == r
    o = masked_softmax_attention(q.view(T, H, d).transpose(0, 1), k.view(T, H, d).transpose(0, 1),
                                 v.view(T, H, e).transpose(0, 1), float(cfg["scale"]), causal_mask(T))
    gate = torch.sigmoid(_r(h @ w[p + "g"].T, round_to))             # [T, H]
    o = _r(o.transpose(0, 1) * gate[:, :, None], round_to).reshape(T, H * e)
    return _r(o @ w[p + "o"].T, round_to)


def chunked_attention(h, w, p, cfg, round_to=None) -> torch.Tensor:
    """Grouped-query attention without positions: scores scaled by the
    config's number and by one learned number per head; keys visible inside
    the query's own chunk of ``mask.size`` positions; sigmoid gate per head."""
    T = h.shape[0]
    H, G, d, e = cfg["heads"], cfg["kv_heads"], cfg["dim"], cfg["vdim"]
    q = _r(h @ w[p + "q"].T, round_to).view(T, H, d).transpose(0, 1)
    k = _r(h @ w[p + "k"].T, round_to).view(T, G, d).transpose(0, 1)
    v = _r(h @ w[p + "v"].T, round_to).view(T, G, e).transpose(0, 1)
    rep = H // G
    k = k.repeat_interleave(rep, dim=0)
    v = v.repeat_interleave(rep, dim=0)
    scale = float(cfg["scale"]) * w[p + "temp"].to(h.dtype)
    visible = chunk_mask(T, int(cfg["mask"]["size"])) if cfg.get("mask") else causal_mask(T)
    o = masked_softmax_attention(q, k, v, scale, visible)
    gate = torch.sigmoid(_r(h @ w[p + "g"].T, round_to))
    o = _r(o.transpose(0, 1) * gate[:, :, None], round_to).reshape(T, H * e)
    return _r(o @ w[p + "o"].T, round_to)


def clamped_glu(h, w, p, cfg, round_to=None) -> torch.Tensor:
    """g = min(gate(h), L); u = clamp(up(h), -L, L); down(g * sigmoid(1.702 g) * (u + 1))."""
    L = float(cfg["limit"])
    g = (h @ w[p + "gate"].T).clamp(max=L)
    u = (h @ w[p + "up"].T).clamp(min=-L, max=L)
    y = _r(g * torch.sigmoid(1.702 * g) * (u + 1.0), round_to)
    return _r(y @ w[p + "down"].T, round_to)


# --------------------------------------------------------------------------
# the model
# --------------------------------------------------------------------------
def forward(cfg: dict, w: dict, ids, dtype=torch.float64, round_to=None, layers_out: list | None = None) -> torch.Tensor:
    """Logits [T, vocab] of a whole sequence.  ``layers_out`` collects the
    residual stream after every layer."""
    w = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in w.items()}
    ids = torch.as_tensor(ids, dtype=torch.long)
    T, W = ids.shape[0], int(cfg["width"])
    eps, groups = float(cfg["norm"]["eps"]), int(cfg["norm"]["groups"])
    x = w["embed"][ids] + sinusoid(torch.arange(T), W, dtype)
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        h = _r(grouped_rmsnorm(x, w[p + "norm1"], eps, groups), round_to)
        if cfg.get("canon"):
            h = _r(causal_taps(h, w[p + "canon1"]), round_to)
        if layer["type"] == "latent_attention":
            x = x + latent_attention(h, w, p + "mix.", layer["mixer"], eps, round_to)
        elif layer["type"] == "attention":
            x = x + chunked_attention(h, w, p + "mix.", layer["mixer"], round_to)
        else:
            raise ValueError(f"unknown layer type {layer['type']!r}")
        if layer.get("mlp") is not None:
            if layer["mlp"]["kind"] != "dense":
                raise ValueError(f"unknown feed-forward kind {layer['mlp']['kind']!r}")
            h = _r(grouped_rmsnorm(x, w[p + "norm2"], eps, groups), round_to)
            x = x + clamped_glu(h, w, p + "mlp.", layer["mlp"], round_to)
        if layers_out is not None:
            layers_out.append(x.clone())
    h = _r(grouped_rmsnorm(x, w["final.norm"], eps, groups), round_to)
    return h @ w["head"].T


def greedy(cfg: dict, w: dict, prompt, steps: int, dtype=torch.float64) -> list[int]:
    ids, out = list(prompt), []
    for _ in range(steps):
        t = int(forward(cfg, w, ids, dtype)[-1].argmax())
        out.append(t)
        ids.append(t)
    return out


# --------------------------------------------------------------------------
# small random models
# --------------------------------------------------------------------------
def tensor_shapes(cfg: dict) -> dict[str, tuple]:
    W, V = int(cfg["width"]), int(cfg["vocab"])
    taps = int(cfg["canon"]["taps"]) if cfg.get("canon") else 0
    shapes = {"embed": (V, W), "final.norm": (W,), "head": (V, W)}
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        shapes[p + "norm1"] = (W,)
        if taps:
            shapes[p + "canon1"] = (W, taps)
        H, d, e = m["heads"], m["dim"], m["vdim"]
        if layer["type"] == "latent_attention":
            r = m["kv_rank"]
            shapes.update({p + "mix.q": (H * d, W), p + "mix.dkv": (r, W), p + "mix.dkv.norm": (r,),
                           p + "mix.uk": (H * d, r), p + "mix.uv": (H * e, r)})
        else:
            G = m["kv_heads"]
            shapes.update({p + "mix.q": (H * d, W), p + "mix.k": (G * d, W), p + "mix.v": (G * e, W),
                           p + "mix.temp": (H,)})
        shapes[p + "mix.g"] = (H, W)
        shapes[p + "mix.o"] = (W, H * e)
        if layer.get("mlp") is not None:
            F = layer["mlp"]["ff"]
            shapes.update({p + "norm2": (W,), p + "mlp.gate": (F, W), p + "mlp.up": (F, W), p + "mlp.down": (W, F)})
    return shapes


def random_weights(cfg: dict, seed: int, std: float | None = None) -> dict[str, torch.Tensor]:
    """bfloat16-representable float32 tensors: matrices N(0, std or 1/sqrt(fan_in)),
    norm weights and per-head numbers around 1, taps around 0."""
    g = torch.Generator().manual_seed(seed)
    out = {}
    for name, shape in tensor_shapes(cfg).items():
        if name.endswith(("norm1", "norm2", "final.norm", "dkv.norm")):
            t = 1.0 + 0.2 * torch.randn(shape, generator=g)
        elif name.endswith("temp"):
            t = 1.0 + 0.5 * torch.rand(shape, generator=g)
        elif name.endswith("canon1"):
            t = 0.3 * torch.randn(shape, generator=g)
        elif name == "embed":
            t = torch.randn(shape, generator=g)
        else:
            t = torch.randn(shape, generator=g) * (std if std is not None else 1.0 / math.sqrt(shape[-1]))
        out[name] = t.to(torch.bfloat16).to(torch.float32)
    return out
