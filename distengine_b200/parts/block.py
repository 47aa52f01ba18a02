"""Pre-norm block: x += mixer(norm(x)); x += feed_forward(norm(x))
(src/models/llama.py:66-89).  The sums are carried as the stream's pending branch and folded in
by the next norm."""

from __future__ import annotations

from .base import Block, register_block
from .context import CacheBinding, ResidualStream, StepContext


class PreNormBlock(Block):
    def forward(self, stream: ResidualStream, ctx: StepContext,
                cache: "CacheBinding | None") -> None:
        h = self.mixer_norm.forward(stream, ctx)
        stream.pending = self.mixer.forward(h, ctx, cache)
        h = self.feed_forward_norm.forward(stream, ctx)
        stream.pending = self.feed_forward.forward(h, ctx)


register_block("prenorm", PreNormBlock)
