"""Arrangement of norms, mixer and feed-forward in a block.

``pre_norm`` is the Llama arrangement (src/cuda/dense_decoder.rs:658-782):

    x  = input_norm(residual [+ pending update])
    a  = mixer(x)
    m  = post_mixer_norm(residual + a)
    f  = feed_forward(m)            -> leaves (residual, f) for the next block's norm

Each addition is fused into the norm that follows it; where the part in front can, its last product does that
norm's work on the way out (``FollowNorm`` -> ``PreparedNorm``), and the product behind only applies the scale.
"""

from __future__ import annotations

from typing import Optional, Tuple

from .base import (BLOCKS, Block, CacheBinding, DeferredNorm, FollowNorm, Norm, PreparedNorm, ResidualStream,
                   StepContext)


@BLOCKS.register("pre_norm")
class PreNormBlock(Block):
    @classmethod
    def norm_roles(cls) -> Tuple[str, ...]:
        return ("input", "post_mixer")

    accepts_next_norm = True

    def entry_norm(self) -> Optional[Norm]:
        return self.norms["input"]

    def forward(self, stream: ResidualStream, ctx: StepContext, cache: Optional[CacheBinding],
                next_norm: Optional[Norm] = None) -> ResidualStream:
        # each norm is handed on unevaluated: a part that can fold it into its first kernel does so
        if stream.prepared is not None and stream.prepared.norm is self.norms["input"]:
            first = stream.prepared                       # the block in front already did this norm's work
        else:
            first = DeferredNorm(self.norms["input"], stream.residual, stream.update)
        x = first if self.mixer.accepts_deferred_norm else first.materialize()
        if self.mixer.accepts_follow_norm:
            mixed = self.mixer.forward(x, ctx, cache, follow=FollowNorm(self.norms["post_mixer"], first))
        else:
            mixed = self.mixer.forward(x, ctx, cache)
        second = mixed if isinstance(mixed, PreparedNorm) else DeferredNorm(self.norms["post_mixer"], first.residual, mixed)
        m = second if self.feed_forward.accepts_deferred_norm else second.materialize()
        if self.feed_forward.accepts_follow_norm and next_norm is not None:
            update = self.feed_forward.forward(m, ctx, follow=FollowNorm(next_norm, second))
        else:
            update = self.feed_forward.forward(m, ctx)
        if isinstance(update, PreparedNorm):
            return ResidualStream(update.residual, None, prepared=update)
        return ResidualStream(second.residual, update)
