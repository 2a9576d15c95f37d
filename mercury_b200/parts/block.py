"""Arrangements: how mixers, a feed-forward and their norms sit in one block.

`PreNormBlock` is mercury/model/qwen2.py:72-94: norm, mixer, norm, feed-forward, with the
residual sum deferred to the next norm. A block receives the residual stream `h` and the
delta that is still to be added to it, and returns the delta it leaves behind.
"""

from __future__ import annotations

from .base import PartSpec, build_part, register_arrangement


class PreNormBlock:
    def __init__(self, mixer: PartSpec, feed_forward: PartSpec, mixer_norm: PartSpec,
                 feed_forward_norm: PartSpec):
        self.mixer = build_part("mixer", mixer)
        self.feed_forward = build_part("feed_forward", feed_forward)
        self.mixer_norm = build_part("norm", mixer_norm)
        self.feed_forward_norm = build_part("norm", feed_forward_norm)

    def mixers(self):
        return [self.mixer]

    def parts(self):
        return [self.mixer_norm, self.mixer, self.feed_forward_norm, self.feed_forward]

    def first_norm(self):
        """The norm that opens this block (what the block before may compute ahead)."""
        return self.mixer_norm

    def forward(self, h, delta, ctx, caches, states, next_norm=None):
        mixer, ff = self.mixer, self.feed_forward
        cache, state = caches[0], states[0]
        x = self.mixer_norm.add_norm(h, delta, ctx,
                                     defer=getattr(mixer, "accepts_pending_norm", False))
        if getattr(mixer, "adds_to_residual", False):
            mixed = mixer.forward(x, ctx, cache, state, residual=h,
                                  then_norm=self.feed_forward_norm)
        else:
            mixed = mixer.forward(x, ctx, cache, state)
        x = self.feed_forward_norm.add_norm(h, mixed, ctx,
                                            defer=getattr(ff, "accepts_pending_norm", False))
        if getattr(ff, "adds_to_residual", False):
            return ff.forward(x, ctx, residual=h, then_norm=next_norm)
        return ff.forward(x, ctx)


register_arrangement("pre_norm", PreNormBlock)
