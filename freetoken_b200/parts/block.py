"""Arrangements of a mixer and a feed-forward around the residual stream.

``prenorm`` is the reference's decoder layer
(python/freetoken/models/minimax_m2/model.py:27-37): the layer receives the
previous branch output ``delta`` and the float32 ``residual``; each norm first
adds the pending branch output into the residual, then normalises::

    h = norm1(delta, residual)      # residual += delta
    a = mixer(h)
    h = norm2(a, residual)          # residual += a
    return feed_forward(h)          # the next norm adds it
"""

from __future__ import annotations

from .base import Block, register_block


@register_block("prenorm")
class PreNormBlock(Block):
    NORM_NAMES = ("mixer", "feed_forward")
    HAS_FEED_FORWARD = True

    def forward(self, ctx, delta, residual, cache):
        h = self.mixer_norm.forward(ctx, delta, residual)
        a = self.mixer.forward(ctx, h, cache)
        h = self.feed_forward_norm.forward(ctx, a, residual)
        return self.feed_forward.forward(ctx, h)
