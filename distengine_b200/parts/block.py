"""Pre-norm block: x += mixer(norm(x)); x += feed_forward(norm(x))
(src/models/llama.py:66-89).  The sums are carried as the stream's pending branch and folded in
by the next norm."""

from __future__ import annotations

from .base import Block, register_block
from .context import CacheBinding, ResidualStream, StepContext


class PreNormBlock(Block):
    def forward(self, stream: ResidualStream, ctx: StepContext, cache: "CacheBinding | None",
                following=None) -> None:
        h = _normed(self.mixer_norm, stream, ctx)
        ahead = _ahead(self.mixer, self.feed_forward_norm, self.feed_forward, stream, ctx)
        if ahead is None:
            stream.pending = self.mixer.forward(h, ctx, cache)
        else:
            self.mixer.forward(h, ctx, cache, ahead=ahead)
            stream.ahead = ahead
        h = _normed(self.feed_forward_norm, stream, ctx)
        ahead = None
        if following is not None:
            ahead = _ahead(self.feed_forward, following[0], following[1], stream, ctx)
        if ahead is None:
            stream.pending = self.feed_forward.forward(h, ctx)
        else:
            self.feed_forward.forward(h, ctx, ahead=ahead)
            stream.ahead = ahead


def _normed(norm, stream: ResidualStream, ctx: StepContext):
    """The norm's output, from the product before it if that did the work."""
    ahead, stream.ahead = stream.ahead, None
    if ahead is None:
        return norm.forward(stream, ctx)
    if ahead.norm is not norm:
        raise RuntimeError("the stream holds another norm's work than the one that runs next")
    return ahead.result()


def _ahead(producer, norm, consumer, stream: ResidualStream, ctx: StepContext):
    """Buffers for ``producer``'s last product to do ``norm``'s work, if producer, norm and
    ``consumer`` (which must take rows without their factors) all can for this step."""
    n = stream.resid.shape[0]
    abilities = (getattr(producer, "ahead_parts", None), getattr(consumer, "takes_unscaled", None))
    if None in abilities:
        return None
    count = abilities[0](n)
    if not count or not abilities[1](n):
        return None
    return norm.ahead(stream, ctx, count)


register_block("prenorm", PreNormBlock)
