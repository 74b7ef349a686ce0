"""A plain, slow implementation of the Kaditar design, one function per
mechanism, whole sequences, no cache, on the CPU.  It shares no code with the
package; the tests compare the package with it.

``round_to`` (a torch dtype or None) is where the serving pipeline rounds
activations between matrix products; everything the design computes in 32 bits
(norms, positions, scores and softmax, routers, the streams) is never rounded.

The design in short.  x_1 .. x_S are S copies of the embedding (S streams).
A sub-layer q of layer l reads u = sum_s a_s x_s, computes y = f(LN(u)) and
writes x_t <- sum_s M[s, t] x_s + b_t y.  f is differential attention (two
softmax maps per head over a sliding window, rotary positions on the leading
dimensions of each map in interleaved pairs, o = A1 v - lam A2 v, normed per
head) or a feed-forward (gated with relu, or routed experts gated with silu
plus a shared expert behind a sigmoid gate).  Some consecutive layers run
several times in a row.  Output: LN of the streams' sum, the embedding matrix
as head, and a tanh cap on the logits.
"""
from __future__ import annotations

import math

import torch


def _r(x, round_to):
    return x if round_to is None else x.to(round_to).to(x.dtype)


def layer_norm(x, weight, bias, eps):
    mean = x.mean(-1, keepdim=True)
    var = ((x - mean) ** 2).mean(-1, keepdim=True)
    return (x - mean) / torch.sqrt(var + eps) * weight + bias


def rotate_pairs(x, positions, rot, base):
    """x [..., T, d]: entries (2i, 2i + 1), i < rot / 2, turn by positions * base^(-2i / rot)."""
    out = x.clone()
    for i in range(rot // 2):
        angle = positions.to(x.dtype) * (base ** (-2.0 * i / rot))
        c, s = torch.cos(angle), torch.sin(angle)
        a, b = x[..., 2 * i], x[..., 2 * i + 1]
        out[..., 2 * i] = a * c - b * s
        out[..., 2 * i + 1] = b * c + a * s
    return out


def window_mask(T, size):
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    return (i - j >= 0) & (i - j < size)


def softmax_attention(q, k, v, scale, visible):
    """q [T, d], k [T, d], v [T, e], visible [T, T] bool."""
    s = (q @ k.T) * scale
    s = s.masked_fill(~visible, float("-inf"))
    return torch.softmax(s, dim=-1) @ v


def differential_lambda(w, p, diff):
    return (math.exp(float((w[p + "lq1"].double() * w[p + "lk1"].double()).sum()))
            - math.exp(float((w[p + "lq2"].double() * w[p + "lk2"].double()).sum())) + diff)


def differential_attention(h, w, p, m, eps, round_to=None):
    """h [T, W]; tensors w[p + ...]; m: the mixer's entry of the config."""
    T = h.shape[0]
    H, G, d, e = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = _r(h @ w[p + "q"].T + w[p + "q.b"], round_to).view(T, H, 2, d)
    k = _r(h @ w[p + "k"].T + w[p + "k.b"], round_to).view(T, G, 2, d)
    v = _r(h @ w[p + "v"].T + w[p + "v.b"], round_to).view(T, G, e)
    pos = torch.arange(T)
    rot, base = (m["rot"]["dims"], m["rot"]["base"]) if m.get("rot") else (0, 1.0)
    q = _r(rotate_pairs(q.permute(1, 2, 0, 3), pos, rot, base), round_to)      # [H, 2, T, d]
    k = _r(rotate_pairs(k.permute(1, 2, 0, 3), pos, rot, base), round_to)      # [G, 2, T, d]
    visible = window_mask(T, m["mask"]["size"]) if m.get("mask") else window_mask(T, T)
    lam = differential_lambda(w, p, m["diff"])
    heads = []
    for head in range(H):
        g = head // (H // G)
        a1 = softmax_attention(q[head, 0], k[g, 0], v[:, g], m["scale"], visible)
        a2 = softmax_attention(q[head, 1], k[g, 1], v[:, g], m["scale"], visible)
        o = a1 - lam * a2
        o = o / torch.sqrt((o * o).mean(-1, keepdim=True) + eps) * (1.0 - m["diff"])
        heads.append(o)
    o = _r(torch.cat(heads, dim=-1), round_to)
    return _r(o @ w[p + "o"].T, round_to)


def gated(h, gate, up, down, act, round_to=None):
    y = _r(act(_r(h @ gate.T, None)) * (h @ up.T), round_to)
    return y @ down.T


def dense_ff(h, w, p, round_to=None):
    return _r(gated(h, w[p + "gate"], w[p + "up"], w[p + "down"], torch.relu, round_to), round_to)


def routed_ff(h, w, p, f, round_to=None):
    """Top experts by router logit, softmax over the chosen logits, plus the
    shared expert times sigmoid(sg . h)."""
    T = h.shape[0]
    E, top = f["router"]["experts"], f["router"]["top"]
    silu = torch.nn.functional.silu
    z = h @ w[p + "router"].T + w[p + "router.b"]
    out = torch.zeros(T, w[p + "e0.down"].shape[0], dtype=h.dtype)
    chosen = torch.topk(z, top, dim=-1)
    share = torch.softmax(chosen.values, dim=-1)
    for t in range(T):
        for j in range(top):
            e = int(chosen.indices[t, j])
            pe = f"{p}e{e}."
            y = _r(gated(h[t:t + 1], w[pe + "gate"], w[pe + "up"], w[pe + "down"], silu, round_to), round_to)
            out[t] += share[t, j] * y[0]
    if f.get("shared") is not None:
        ps = p + "shared."
        y = _r(gated(h, w[ps + "gate"], w[ps + "up"], w[ps + "down"], silu, round_to), round_to)
        out = out + torch.sigmoid(h @ w[ps + "sg"].T) * y
    return _r(out, round_to) if round_to is not None else out


def run_order(cfg):
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop:
        return list(range(n))
    body = list(range(loop["start"], loop["stop"]))
    return list(range(loop["start"])) + body * loop["times"] + list(range(loop["stop"], n))


def forward(cfg, w, ids, dtype=torch.float64, round_to=None, layers_out=None):
    """Logits [T, vocab] for one whole sequence.  ``layers_out`` (a list)
    receives the sum of the streams after every layer run."""
    w = {k: v.to(dtype) if v.is_floating_point() else v for k, v in w.items()}
    ids = torch.as_tensor(ids, dtype=torch.long)
    eps = cfg["norm"]["eps"]
    S = cfg.get("streams")
    x0 = w["embed"][ids]
    streams = [x0.clone() for _ in range(S)] if S else None
    x = x0

    def sublayer(x, streams, p, q, f):
        if streams is None:
            return x + f(_r(layer_norm(x, w[f"{p}norm{q}"], w[f"{p}norm{q}.b"], eps), round_to)), None
        a, b, M = w[f"{p}hc{q}.in"], w[f"{p}hc{q}.out"], w[f"{p}hc{q}.mix"]
        u = sum(a[s] * streams[s] for s in range(S))
        y = f(_r(layer_norm(u, w[f"{p}norm{q}"], w[f"{p}norm{q}.b"], eps), round_to))
        new = [sum(M[s, t] * streams[s] for s in range(S)) + b[t] * y for t in range(S)]
        return None, new

    for i in run_order(cfg):
        layer = cfg["layers"][i]
        p = f"l{i}."
        x, streams = sublayer(x, streams, p, 1,
                              lambda h: differential_attention(h, w, p + "mix.", layer["mixer"], eps, round_to))
        f = layer.get("mlp")
        if f is not None:
            if f["kind"] == "dense":
                x, streams = sublayer(x, streams, p, 2, lambda h: dense_ff(h, w, p + "mlp.", round_to))
            else:
                x, streams = sublayer(x, streams, p, 2, lambda h: routed_ff(h, w, p + "mlp.", f, round_to))
        if layers_out is not None:
            layers_out.append(sum(streams) if streams is not None else x)
    if streams is not None:
        x = sum(streams)
    h = _r(layer_norm(x, w["final.norm"], w["final.norm.b"], eps), round_to)
    logits = h @ w["embed"].T
    cap = cfg.get("logit_softcap")
    return cap * torch.tanh(logits / cap) if cap else logits


def greedy(cfg, w, prompt, steps, dtype=torch.float64):
    ids = list(prompt)
    out = []
    for _ in range(steps):
        nxt = int(torch.argmax(forward(cfg, w, ids, dtype)[-1]))
        out.append(nxt)
        ids.append(nxt)
    return out


def tensor_shapes(cfg):
    W, V = cfg["width"], cfg["vocab"]
    S = cfg.get("streams")
    shapes = {"embed": (V, W), "final.norm": (W,), "final.norm.b": (W,)}
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        m = layer["mixer"]
        H, G, d, e = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
        shapes.update({p + "norm1": (W,), p + "norm1.b": (W,),
                       p + "mix.q": (H * 2 * d, W), p + "mix.q.b": (H * 2 * d,), p + "mix.k": (G * 2 * d, W),
                       p + "mix.k.b": (G * 2 * d,), p + "mix.v": (G * e, W), p + "mix.v.b": (G * e,),
                       p + "mix.lq1": (d,), p + "mix.lk1": (d,), p + "mix.lq2": (d,), p + "mix.lk2": (d,),
                       p + "mix.o": (W, H * e)})
        subs = [1]
        f = layer.get("mlp")
        if f is not None:
            subs.append(2)
            shapes.update({p + "norm2": (W,), p + "norm2.b": (W,)})
            if f["kind"] == "dense":
                shapes.update({p + "mlp.gate": (f["ff"], W), p + "mlp.up": (f["ff"], W), p + "mlp.down": (W, f["ff"])})
            else:
                E, ff = f["router"]["experts"], f["expert"]["ff"]
                shapes.update({p + "mlp.router": (E, W), p + "mlp.router.b": (E,)})
                for e_ in range(E):
                    shapes.update({f"{p}mlp.e{e_}.gate": (ff, W), f"{p}mlp.e{e_}.up": (ff, W), f"{p}mlp.e{e_}.down": (W, ff)})
                if f.get("shared") is not None:
                    sf = f["shared"]["ff"]
                    shapes.update({p + "mlp.shared.gate": (sf, W), p + "mlp.shared.up": (sf, W),
                                   p + "mlp.shared.down": (W, sf), p + "mlp.shared.sg": (1, W)})
        if S:
            for q in subs:
                shapes.update({f"{p}hc{q}.in": (S,), f"{p}hc{q}.out": (S,), f"{p}hc{q}.mix": (S, S)})
    return shapes


def random_weights(cfg, seed, std=None):
    """Weights that keep activations of order one and make every mechanism
    count: norm biases and projection biases away from zero, mix matrices near
    the identity with real off-diagonal entries, lambda vectors that give a
    lambda of order one, router biases that spread the choice of experts."""
    g = torch.Generator().manual_seed(seed)
    W = cfg["width"]
    out = {}
    for name, shape in tensor_shapes(cfg).items():
        leaf = name.split(".")[-1]
        if name.endswith(".b") and "norm" in name:
            t = 0.1 * torch.randn(shape, generator=g)
        elif "norm" in name:
            t = 1.0 + 0.1 * torch.randn(shape, generator=g)
        elif name.endswith(".b"):
            t = 0.3 * torch.randn(shape, generator=g)
        elif leaf in ("lq1", "lk1", "lq2", "lk2"):
            t = 0.3 * torch.randn(shape, generator=g)
        elif leaf == "in":
            t = 1.0 / shape[0] + 0.2 * torch.randn(shape, generator=g)
        elif leaf == "out":
            t = 1.0 + 0.3 * torch.randn(shape, generator=g)
        elif leaf == "mix" and len(shape) == 2 and ".hc" in name:
            t = torch.eye(shape[0]) + 0.15 * torch.randn(shape, generator=g)
        elif name == "embed":
            t = torch.randn(shape, generator=g)
        else:
            s = std if std is not None else 1.0 / math.sqrt(shape[-1])
            t = s * torch.randn(shape, generator=g)
        out[name] = t.to(torch.bfloat16).float()      # values both storage types hold exactly
    return out
