"""Arrangements of a layer's parts around the residual stream.

`pre_norm` (student_engine.py:696-731):  h += mixer(norm_1(h));  h += feed_forward(norm_2(h)).
The stream `hidden` is float32 and is updated in place; a part's output (`delta`) is added to it by
the *next* norm's kernel, so a block takes the pending delta of the layer before it and returns its own."""
from __future__ import annotations

from .base import Part
from .registry import build_part, register_part


class PreNormBlock(Part):
    """Reads the layer spec's parts `mixer_norm`, `mixer`, `feed_forward_norm`, `feed_forward`."""

    def __init__(self, layer_spec):
        self.kind = "pre_norm"
        self.mixer_norm = build_part("norm", layer_spec.part("mixer_norm"))
        self.mixer = build_part("mixer", layer_spec.part("mixer"))
        self.feed_forward_norm = build_part("norm", layer_spec.part("feed_forward_norm"))
        self.feed_forward = build_part("feed_forward", layer_spec.part("feed_forward"))

    def sub_parts(self):
        return [self.mixer_norm, self.mixer, self.feed_forward_norm, self.feed_forward]

    def cache_need(self):
        return self.mixer.cache_need()

    def forward(self, hidden, delta, ctx, site, writes_cache):
        rms = self.mixer_norm.fused_rms()
        if rms is not None and self.mixer.fused_takes(ctx):
            self.mixer.fused_forward(hidden, rms, ctx, site, writes_cache, delta)
            delta = None
        else:
            x = self.mixer_norm.forward(hidden, delta)
            delta = self.mixer.forward(x, ctx, site, writes_cache)
        rms = self.feed_forward_norm.fused_rms()
        if rms is not None and self.feed_forward.fused_takes(ctx):
            self.feed_forward.fused_forward(hidden, rms, ctx, delta)
            return None
        x = self.feed_forward_norm.forward(hidden, delta)
        return self.feed_forward.forward(x, ctx)


register_part("block", "pre_norm", PreNormBlock)
