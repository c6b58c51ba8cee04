"""Arrangement of norms, mixer and feed-forward in a block.

``pre_norm`` is the Llama arrangement (src/cuda/dense_decoder.rs:658-782):

    x  = input_norm(residual [+ pending update])
    a  = mixer(x)
    m  = post_mixer_norm(residual + a)
    f  = feed_forward(m)            -> leaves (residual, f) for the next block's norm

Each addition is fused into the norm that follows it.
"""

from __future__ import annotations

from typing import Optional, Tuple

from .base import BLOCKS, Block, CacheBinding, ResidualStream, StepContext


@BLOCKS.register("pre_norm")
class PreNormBlock(Block):
    @classmethod
    def norm_roles(cls) -> Tuple[str, ...]:
        return ("input", "post_mixer")

    def forward(self, stream: ResidualStream, ctx: StepContext, cache: Optional[CacheBinding]) -> ResidualStream:
        residual = stream.residual
        if stream.update is None:
            x = self.norms["input"].forward(residual)
        else:
            x = self.norms["input"].forward_add(residual, stream.update)
        mixed = self.mixer.forward(x, ctx, cache)
        m = self.norms["post_mixer"].forward_add(residual, mixed)
        update = self.feed_forward.forward(m, ctx)
        return ResidualStream(residual, update)
