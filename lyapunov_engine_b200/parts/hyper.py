"""A block arrangement that keeps the residual stream in several copies
("hyper-connections").

Each sub-layer q (the mixer, the feed-forward) has a link with three small
tensors: ``pre`` [S], ``post`` [S] and ``mix`` [S, S] (indexed [from, to]).  It
reads u = sum_s pre[s] x_s, computes y = f(norm(u)), and every copy becomes,
all from the old ones, x_t <- sum_s mix[s, t] x_s + post[t] y.  All copies start
as the embedding's output; what follows the last layer reads their sum.  The
update is not a launch of its own: a sub-layer leaves y pending with its link,
and the next norm's kernel applies it before it reads (``Norm.apply_stream``).
S = 1 is allowed (one copy with a factor on every path).
"""
from __future__ import annotations

from .base import FEED_FORWARDS, MIXERS, NORMS, Block, Part, PartSpec, TensorDecl, register_block


class StreamLink(Part):
    """The three tensors of one sub-layer's link to the copies, kept in 32 bits."""

    def __init__(self, copies: int, pre_name: str, post_name: str, mix_name: str):
        self.copies = int(copies)
        self.names = (pre_name, post_name, mix_name)
        self.pre = self.post = self.mix = None

    def tensors(self):
        pre, post, mix = self.names
        S = self.copies
        return [TensorDecl(pre, (S,), role="vector", init="share"), TensorDecl(post, (S,), role="vector", init="ones"),
                TensorDecl(mix, (S, S), role="vector", init="eye")]

    def bind(self, get, runtime):
        self.pre, self.post, self.mix = (get(n).contiguous() for n in self.names)


@register_block("hyper_prenorm")
class HyperPreNormBlock(Block):
    def __init__(self, copies: int, mixer: PartSpec, feed_forward: PartSpec | None, mixer_norm: PartSpec,
                 feed_forward_norm: PartSpec | None, mixer_link: dict, feed_forward_link: dict | None):
        if (feed_forward is None) != (feed_forward_norm is None) or (feed_forward is None) != (feed_forward_link is None):
            raise ValueError("a block has a feed-forward with its norm and its link, or none of them")
        self.copies = int(copies)
        if not 1 <= self.copies <= 8:
            raise ValueError(f"the residual stream is kept in 1 to 8 copies, got {copies}")
        self.mixer = MIXERS.build(mixer)
        self.feed_forward = FEED_FORWARDS.build(feed_forward) if feed_forward is not None else None
        self.mixer_norm = NORMS.build(mixer_norm)
        self.feed_forward_norm = NORMS.build(feed_forward_norm) if feed_forward_norm is not None else None
        self.mixer_link = StreamLink(self.copies, **mixer_link)
        self.feed_forward_link = StreamLink(self.copies, **feed_forward_link) if feed_forward_link is not None else None

    def parts(self):
        return [p for p in (self.mixer_norm, self.mixer_link, self.mixer, self.feed_forward_norm, self.feed_forward_link,
                            self.feed_forward) if p is not None]

    def tensors(self):
        return [d for p in self.parts() for d in p.tensors()]

    def bind(self, get, runtime):
        for p in self.parts():
            p.bind(get, runtime)

    def forward(self, stream, ctx, cache) -> None:
        n = self.mixer_norm.apply_stream(stream, read=self.mixer_link, workspace=ctx.workspace)
        stream.pending = self.mixer.forward(n, ctx, cache)
        stream.update = self.mixer_link
        if self.feed_forward is None:
            return
        n = self.feed_forward_norm.apply_stream(stream, read=self.feed_forward_link, workspace=ctx.workspace)
        stream.pending = self.feed_forward.forward(n, ctx)
        stream.update = self.feed_forward_link
