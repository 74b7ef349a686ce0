"""The Kaditar decoder as a description: which parts, with which numbers and
tensor names, in which order.

Token embedding; layers of a pre-norm arrangement over a residual stream kept
in ``streams`` copies (hyper-connections; without the key, one stream with
plain additions), norms with weight and bias; the mixer is differential
attention (two maps per head, rotary positions on neighbouring pairs, a
sliding window, biases); the feed-forward is gated with relu, or routed experts
gated with silu plus a shared expert behind a sigmoid gate; a stretch of
consecutive layers may run several times in a row, each pass with a cache of
its own (the run order names those layers again); the last norm reads the sum
of the copies; the head is the embedding matrix, and the logits are capped by a
tanh.  Tensor names: ``embed``, ``l<i>.norm1|norm2[.b]``, ``l<i>.mix.*``,
``l<i>.mlp.*``, ``l<i>.hc1|hc2.in|out|mix``, ``final.norm[.b]``.
"""
from __future__ import annotations

from ..config.kaditar import KaditarConfig
from ..parts.base import LayerSpec, ModelSpec, PartSpec, RunSpec

# Positions are computed, not looked up: the limit is where a float32 stops counting exactly.
MAX_POSITIONS = 1 << 24


def kaditar_spec(raw_config: dict) -> ModelSpec:
    c = KaditarConfig.from_dict(raw_config)
    W = c.width

    def norm(name):
        return PartSpec("layernorm", {"hidden_size": W, "eps": c.norm_eps, "weight_name": name, "bias_name": name + ".b"})

    def link(prefix):
        return {"pre_name": prefix + ".in", "post_name": prefix + ".out", "mix_name": prefix + ".mix"}

    def gated(kind, prefix, ff):
        return PartSpec(kind, {"hidden_size": W, "intermediate_size": ff, "gate_name": prefix + "gate",
                               "up_name": prefix + "up", "down_name": prefix + "down"})

    layers = []
    for i, layer in enumerate(c.layers):
        p = f"l{i}."
        m = layer.mixer
        mixer = PartSpec("differential_attention", {
            "hidden_size": W, "num_heads": m.heads, "num_kv_heads": m.kv_heads, "head_dim": m.dim, "value_dim": m.vdim,
            "scale": m.scale, "diff": m.diff, "norm_eps": c.norm_eps, "rot": m.rot_dims, "rot_base": m.rot_base,
            "window": m.window or None, "q_name": p + "mix.q", "k_name": p + "mix.k", "v_name": p + "mix.v",
            "o_name": p + "mix.o", "bias_names": (p + "mix.q.b", p + "mix.k.b", p + "mix.v.b"),
            "lambda_names": (p + "mix.lq1", p + "mix.lk1", p + "mix.lq2", p + "mix.lk2")})
        feed_forward = None
        f = layer.feed_forward
        if f is not None and f.kind == "dense":
            feed_forward = gated("gated_relu", p + "mlp.", f.ff)
        elif f is not None:
            feed_forward = PartSpec("routed_experts", {
                "hidden_size": W, "intermediate_size": f.ff, "num_experts": f.experts, "top": f.top,
                "router_name": p + "mlp.router", "router_bias_name": p + "mlp.router.b",
                "expert_names": p + "mlp.e{expert}.{part}", "activation": "silu",
                "shared": gated("gated_silu", p + "mlp.shared.", f.shared_ff) if f.shared_ff else None,
                "shared_gate_name": p + "mlp.shared.sg" if f.shared_ff else None})
        ff_norm = norm(p + "norm2") if feed_forward is not None else None
        if c.streams:
            block = PartSpec("hyper_prenorm", {
                "copies": c.streams, "mixer": mixer, "feed_forward": feed_forward, "mixer_norm": norm(p + "norm1"),
                "feed_forward_norm": ff_norm, "mixer_link": link(p + "hc1"),
                "feed_forward_link": link(p + "hc2") if feed_forward is not None else None})
        else:
            block = PartSpec("prenorm", {"mixer": mixer, "feed_forward": feed_forward, "mixer_norm": norm(p + "norm1"),
                                         "feed_forward_norm": ff_norm})
        layers.append(LayerSpec(block))
    return ModelSpec(
        architecture=c.architecture,
        hidden_size=W,
        vocab_size=c.vocab,
        max_positions=MAX_POSITIONS,
        embedding=PartSpec("token_embedding", {"vocab_size": c.vocab, "hidden_size": W, "weight_name": "embed"}),
        layers=tuple(layers),
        run_order=tuple(RunSpec(i) for i in c.run_order()),
        final_norm=norm("final.norm"),
        head=PartSpec("linear_head", {"vocab_size": c.vocab, "hidden_size": W, "weight_name": "embed", "tied_to": None,
                                      "softcap": c.logit_softcap or None}),
        config_json=dict(c.raw),
    )
