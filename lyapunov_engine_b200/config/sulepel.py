"""SulepelConfig: the keys of a Sulepel checkpoint's config.json, typed.

A Sulepel model is a list of layers, each with a mixer of its own kind and
sizes and an optional feed-forward; one grouped RMS norm and one short
convolution setting serve all layers.  Every size and constant is read from the
file; nothing has a default.

    {"architecture": "Sulepel", "vocab": V, "width": W,
     "norm": {"eps": .., "groups": ..}, "canon": {"taps": ..},
     "layers": [{"type": "latent_attention" | "attention",
                 "mixer": {...}, "mlp": {"kind": "dense", "ff": .., "limit": ..} | null}, ...]}
"""
from __future__ import annotations

from dataclasses import dataclass

from .base import ConfigError, KeyReader


@dataclass(frozen=True)
class SulepelFeedForward:
    kind: str
    ff: int
    limit: float


@dataclass(frozen=True)
class SulepelMixer:
    """``kind`` "latent_attention": heads, dim, vdim, kv_rank, scale;
    "attention": heads, kv_heads, dim, vdim, scale, chunk (``mask.size``)."""
    kind: str
    heads: int
    dim: int
    vdim: int
    scale: float
    kv_rank: int = 0
    kv_heads: int = 0
    chunk: int = 0


@dataclass(frozen=True)
class SulepelLayer:
    mixer: SulepelMixer
    feed_forward: SulepelFeedForward | None


@dataclass(frozen=True)
class SulepelConfig:
    architecture: str
    vocab: int
    width: int
    norm_eps: float
    norm_groups: int
    taps: int                      # 0: no input convolution
    layers: tuple[SulepelLayer, ...]
    raw: dict

    @staticmethod
    def from_dict(raw: dict, source: str = "config.json") -> "SulepelConfig":
        r = KeyReader(raw, source)
        width = r.integer("width")
        norm = KeyReader(r.mapping("norm"), source + ": norm")
        # (a config without "canon" describes a model without the input convolution)
        raw_canon = r.mapping("canon", None)
        canon = KeyReader(raw_canon if raw_canon is not None else {"taps": 0}, source + ": canon")
        groups = norm.integer("groups")
        if width % groups:
            raise ConfigError(f"{source}: width {width} does not divide into norm.groups {groups}")
        entries = raw.get("layers")
        if not isinstance(entries, list) or not entries:
            raise ConfigError(f"{source}: 'layers' must be a non-empty list")
        layers = []
        for i, entry in enumerate(entries):
            where = f"{source}: layers[{i}]"
            if not isinstance(entry, dict):
                raise ConfigError(f"{where} must be an object")
            e = KeyReader(entry, where)
            kind = e.string("type")
            m = KeyReader(e.mapping("mixer"), where + ".mixer")
            if kind == "latent_attention":
                mixer = SulepelMixer(kind, m.integer("heads"), m.integer("dim"), m.integer("vdim"),
                                     m.number("scale", positive=False), kv_rank=m.integer("kv_rank"))
            elif kind == "attention":
                # (a mixer without "mask" sees every earlier key)
                mask = m.mapping("mask", None)
                chunk = KeyReader(mask, where + ".mixer.mask").integer("size") if mask is not None else 0
                mixer = SulepelMixer(kind, m.integer("heads"), m.integer("dim"), m.integer("vdim"),
                                     m.number("scale", positive=False), kv_heads=m.integer("kv_heads"), chunk=chunk)
                if mixer.heads % mixer.kv_heads:
                    raise ConfigError(f"{where}.mixer: {mixer.heads} heads do not divide into {mixer.kv_heads} kv_heads")
            else:
                raise ConfigError(f"{where}: unknown layer type {kind!r} (known: 'latent_attention', 'attention')")
            ff = None
            if entry.get("mlp") is not None:
                f = KeyReader(e.mapping("mlp"), where + ".mlp")
                ff_kind = f.string("kind")
                if ff_kind != "dense":
                    raise ConfigError(f"{where}.mlp: unknown kind {ff_kind!r} (known: 'dense')")
                ff = SulepelFeedForward(ff_kind, f.integer("ff"), f.number("limit"))
            layers.append(SulepelLayer(mixer, ff))
        return SulepelConfig(architecture=r.string("architecture"), vocab=r.integer("vocab"), width=width,
                             norm_eps=norm.number("eps"), norm_groups=groups, taps=canon.integer("taps", minimum=0),
                             layers=tuple(layers), raw=dict(raw))
