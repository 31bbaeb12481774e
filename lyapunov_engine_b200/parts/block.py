"""Block arrangements: how norms, mixer and feed-forward sit around the
residual stream.

"prenorm" is the reference's decoder layer
(python/lyapunov_engine/models/llama.py:136-165):
    h = h + mixer(norm1(h));  h = h + feed_forward(norm2(h))
The additions happen inside the following norm's kernel, in 32 bits: a block
leaves its feed-forward output ``pending`` and the next norm (of the next
block, or the final one) adds it.
"""
from __future__ import annotations

from .base import BLOCKS, FEED_FORWARDS, MIXERS, NORMS, Block, PartSpec, register_block


@register_block("prenorm")
class PreNormBlock(Block):
    def __init__(self, mixer: PartSpec, feed_forward: PartSpec, mixer_norm: PartSpec, feed_forward_norm: PartSpec):
        self.mixer = MIXERS.build(mixer)
        self.feed_forward = FEED_FORWARDS.build(feed_forward)
        self.mixer_norm = NORMS.build(mixer_norm)
        self.feed_forward_norm = NORMS.build(feed_forward_norm)

    def parts(self):
        return [self.mixer_norm, self.mixer, self.feed_forward_norm, self.feed_forward]

    def tensors(self):
        return [d for p in self.parts() for d in p.tensors()]

    def bind(self, get, runtime):
        for p in self.parts():
            p.bind(get, runtime)

    def forward(self, stream, ctx, cache) -> None:
        n = self.mixer_norm.apply(stream.resid, stream.pending, workspace=ctx.workspace)
        a = self.mixer.forward(n, ctx, cache)
        n = self.feed_forward_norm.apply(stream.resid, a, workspace=ctx.workspace)
        stream.pending = self.feed_forward.forward(n, ctx)
