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

from .base import BLOCKS, Block, CacheBinding, DeferredNorm, ResidualStream, StepContext


@BLOCKS.register("pre_norm")
class PreNormBlock(Block):
    @classmethod
    def norm_roles(cls) -> Tuple[str, ...]:
        return ("input", "post_mixer")

    def forward(self, stream: ResidualStream, ctx: StepContext, cache: Optional[CacheBinding]) -> ResidualStream:
        # each norm is handed on unevaluated: a part that can fold it into its first kernel does so
        first = DeferredNorm(self.norms["input"], stream.residual, stream.update)
        x = first if self.mixer.accepts_deferred_norm else first.materialize()
        mixed = self.mixer.forward(x, ctx, cache)
        second = DeferredNorm(self.norms["post_mixer"], first.residual, mixed)
        m = second if self.feed_forward.accepts_deferred_norm else second.materialize()
        update = self.feed_forward.forward(m, ctx)
        return ResidualStream(second.residual, update)
