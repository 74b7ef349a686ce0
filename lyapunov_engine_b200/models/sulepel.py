"""The Sulepel decoder as a description: which parts, with which numbers and
tensor names, in which order.

Token embedding plus a fixed sinusoidal position vector; per layer a pre-norm
block whose norms are RMS norms in groups, whose mixer reads the first norm's
output through a short causal convolution (``l<i>.canon1``) and is either
latent attention (one cached latent per token, no positions) or grouped-query
attention without positions over chunks of the sequence with a learned factor
per head, both with a sigmoid gate per head; an optional feed-forward with the
clamped gated activation; the same grouped norm before a linear head.  Tensor
names: ``embed``, ``l<i>.norm1|norm2|canon1``, ``l<i>.mix.*``, ``l<i>.mlp.*``,
``final.norm``, ``head``.
"""
from __future__ import annotations

from ..config.sulepel import SulepelConfig
from ..parts.base import LayerSpec, ModelSpec, PartSpec, RunSpec

# Positions are computed, not looked up: the limit is where a float32 stops counting exactly.
MAX_POSITIONS = 1 << 24
SINUSOID_BASE = 10000.0
ACTIVATION_SLOPE = 1.702


def sulepel_spec(raw_config: dict) -> ModelSpec:
    c = SulepelConfig.from_dict(raw_config)
    W = c.width

    def norm(name):
        return PartSpec("rmsnorm", {"hidden_size": W, "eps": c.norm_eps, "weight_name": name, "groups": c.norm_groups})

    layers = []
    for i, layer in enumerate(c.layers):
        p = f"l{i}."
        m = layer.mixer
        if m.kind == "latent_attention":
            mixer = PartSpec("latent_attention", {
                "hidden_size": W, "num_heads": m.heads, "head_dim": m.dim, "value_dim": m.vdim, "latent_dim": m.kv_rank,
                "scale": m.scale, "norm_eps": c.norm_eps, "q_name": p + "mix.q", "down_name": p + "mix.dkv",
                "latent_norm_name": p + "mix.dkv.norm", "up_k_name": p + "mix.uk", "up_v_name": p + "mix.uv",
                "o_name": p + "mix.o", "gate_name": p + "mix.g"})
        else:
            mixer = PartSpec("attention", {
                "hidden_size": W, "num_heads": m.heads, "num_kv_heads": m.kv_heads, "head_dim": m.dim,
                "value_dim": m.vdim, "position": None, "scale": m.scale, "chunk": m.chunk or None,
                "q_name": p + "mix.q", "k_name": p + "mix.k", "v_name": p + "mix.v", "o_name": p + "mix.o",
                "head_scale_name": p + "mix.temp", "gate_name": p + "mix.g"})
        feed_forward = feed_forward_norm = None
        if layer.feed_forward is not None:
            f = layer.feed_forward
            feed_forward = PartSpec("gated_clamped", {
                "hidden_size": W, "intermediate_size": f.ff, "gate_name": p + "mlp.gate", "up_name": p + "mlp.up",
                "down_name": p + "mlp.down", "limit": f.limit, "slope": ACTIVATION_SLOPE})
            feed_forward_norm = norm(p + "norm2")
        layers.append(LayerSpec(PartSpec("prenorm", {
            "mixer": mixer, "feed_forward": feed_forward, "mixer_norm": norm(p + "norm1"),
            "feed_forward_norm": feed_forward_norm,
            "mixer_input": (PartSpec("causal_taps", {"channels": W, "taps": c.taps, "weight_name": p + "canon1"})
                            if c.taps else None)})))
    return ModelSpec(
        architecture=c.architecture,
        hidden_size=W,
        vocab_size=c.vocab,
        max_positions=MAX_POSITIONS,
        embedding=PartSpec("token_embedding_sinusoid", {"vocab_size": c.vocab, "hidden_size": W, "weight_name": "embed",
                                                         "base": SINUSOID_BASE}),
        layers=tuple(layers),
        run_order=tuple(RunSpec(i) for i in range(len(layers))),
        final_norm=norm("final.norm"),
        head=PartSpec("linear_head", {"vocab_size": c.vocab, "hidden_size": W, "weight_name": "head", "tied_to": None}),
        config_json=dict(c.raw),
    )
