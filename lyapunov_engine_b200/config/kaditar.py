"""KaditarConfig: the keys of a Kaditar checkpoint's config.json, typed.

    {"architecture": "Kaditar", "vocab": V, "width": W, "norm": {"eps": ..},
     "streams": S, "logit_softcap": c, "loop": {"start": a, "stop": b, "times": n},
     "layers": [{"type": "attention",
                 "mixer": {"heads", "kv_heads", "dim", "vdim", "scale", "diff",
                           "rot": {"dims", "base"}, "mask": {"size"}},
                 "mlp": {"kind": "dense", "ff": ..}
                      | {"kind": "moe", "expert": {"ff"}, "router": {"experts", "top"}, "shared": {"ff"}}
                      | null}, ...]}

Every size and constant a layer uses is read from its own entry; nothing has a
default.  Keys that may be absent, and what their absence means: ``streams``
(one residual stream with plain additions), ``loop`` (every layer runs once),
``logit_softcap`` (no cap), a mixer's ``mask`` (every earlier key is visible)
and ``rot`` (no position encoding), a routed feed-forward's ``shared`` (no
shared expert), ``mlp`` null (a layer without feed-forward).
"""
from __future__ import annotations

from dataclasses import dataclass

from .base import ConfigError, KeyReader


@dataclass(frozen=True)
class KaditarMixer:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    diff: float
    rot_dims: int          # 0: no rotary encoding
    rot_base: float
    window: int            # 0: every earlier key


@dataclass(frozen=True)
class KaditarFeedForward:
    kind: str              # "dense" or "moe"
    ff: int                # of the dense layer, or of one expert
    experts: int = 0
    top: int = 0
    shared_ff: int = 0     # 0: no shared expert


@dataclass(frozen=True)
class KaditarLayer:
    mixer: KaditarMixer
    feed_forward: KaditarFeedForward | None


@dataclass(frozen=True)
class KaditarConfig:
    architecture: str
    vocab: int
    width: int
    norm_eps: float
    streams: int                       # 0: a single stream with plain additions
    logit_softcap: float               # 0: none
    loop: tuple[int, int, int] | None  # (start, stop, times)
    layers: tuple[KaditarLayer, ...]
    raw: dict

    def run_order(self) -> list[int]:
        n = len(self.layers)
        if self.loop is None:
            return list(range(n))
        start, stop, times = self.loop
        return list(range(start)) + list(range(start, stop)) * times + list(range(stop, n))

    @staticmethod
    def from_dict(raw: dict, source: str = "config.json") -> "KaditarConfig":
        r = KeyReader(raw, source)
        width = r.integer("width")
        norm = KeyReader(r.mapping("norm"), source + ": norm")
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
            if kind != "attention":
                raise ConfigError(f"{where}: unknown layer type {kind!r} (known: 'attention')")
            m = KeyReader(e.mapping("mixer"), where + ".mixer")
            rot = m.mapping("rot", None)
            rot_dims, rot_base = 0, 1.0
            if rot is not None:
                rr = KeyReader(rot, where + ".mixer.rot")
                rot_dims, rot_base = rr.integer("dims", minimum=0), rr.number("base")
            mask = m.mapping("mask", None)
            window = KeyReader(mask, where + ".mixer.mask").integer("size") if mask is not None else 0
            mixer = KaditarMixer(heads=m.integer("heads"), kv_heads=m.integer("kv_heads"), dim=m.integer("dim"),
                                 vdim=m.integer("vdim"), scale=m.number("scale"), diff=m.number("diff", positive=False),
                                 rot_dims=rot_dims, rot_base=rot_base, window=window)
            if mixer.heads % mixer.kv_heads:
                raise ConfigError(f"{where}.mixer: {mixer.heads} heads do not divide into {mixer.kv_heads} kv_heads")
            if mixer.rot_dims % 2 or mixer.rot_dims > mixer.dim:
                raise ConfigError(f"{where}.mixer.rot: dims {mixer.rot_dims} must be even and at most dim {mixer.dim}")
            ff = None
            if entry.get("mlp") is not None:
                f = KeyReader(e.mapping("mlp"), where + ".mlp")
                ff_kind = f.string("kind")
                if ff_kind == "dense":
                    ff = KaditarFeedForward("dense", f.integer("ff"))
                elif ff_kind == "moe":
                    router = KeyReader(f.mapping("router"), where + ".mlp.router")
                    shared = f.mapping("shared", None)
                    ff = KaditarFeedForward("moe", KeyReader(f.mapping("expert"), where + ".mlp.expert").integer("ff"),
                                            experts=router.integer("experts"), top=router.integer("top"),
                                            shared_ff=KeyReader(shared, where + ".mlp.shared").integer("ff") if shared is not None else 0)
                    if ff.top > ff.experts:
                        raise ConfigError(f"{where}.mlp.router: top {ff.top} of {ff.experts} experts")
                else:
                    raise ConfigError(f"{where}.mlp: unknown kind {ff_kind!r} (known: 'dense', 'moe')")
            layers.append(KaditarLayer(mixer, ff))
        loop = None
        raw_loop = r.mapping("loop", None)
        if raw_loop is not None:
            lp = KeyReader(raw_loop, source + ": loop")
            loop = (lp.integer("start", minimum=0), lp.integer("stop", minimum=0), lp.integer("times", minimum=0))
            if not loop[0] <= loop[1] <= len(layers):
                raise ConfigError(f"{source}: loop {loop[0]}..{loop[1]} does not lie within the {len(layers)} layers")
        return KaditarConfig(architecture=r.string("architecture"), vocab=r.integer("vocab"), width=width,
                             norm_eps=norm.number("eps"), streams=r.integer("streams", 0, minimum=0),
                             logit_softcap=r.number("logit_softcap", 0.0, positive=False), loop=loop, layers=tuple(layers),
                             raw=dict(raw))
