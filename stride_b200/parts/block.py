"""Arrangement of parts in a layer. ``pre_norm``: the mixer and the feed-forward
each read a normed copy of the residual stream and add their output back
(python/stride_worker/model.py:254-310)."""

from __future__ import annotations

from .base import Layer, build_part, register_part


class PreNormLayer(Layer):
    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        self.mixer_norm = build_part("norm", spec.mixer_norm, runtime)
        self.mixer = build_part("mixer", spec.mixer, runtime)
        self.ffn_norm = build_part("norm", spec.ffn_norm, runtime)
        self.feed_forward = build_part("feed_forward", spec.feed_forward, runtime)

    def parts(self):
        return (self.mixer_norm, self.mixer, self.ffn_norm, self.feed_forward)

    def declare(self):
        d = {}
        for p in self.parts():
            d.update(p.declare())
        return d

    def bind(self, weights):
        for p in self.parts():
            p.bind(weights)

    def named_tensors(self):
        d = {}
        for p in self.parts():
            d.update(p.named_tensors())
        return d

    def forward(self, stream, ctx, cache):
        # A part that can, gets the norm folded into its first product and leaves its last product to the stream,
        # which folds it into the next norm (decode steps in bfloat16; everything else runs part by part).
        mixer, ffn = self.mixer, self.feed_forward
        h = stream.normed(self.mixer_norm, fold_ok=mixer.accepts_folded)
        stream.add(mixer.forward(h, ctx, cache, lazy_output=True) if mixer.lazy_output else mixer.forward(h, ctx, cache))
        h = stream.normed(self.ffn_norm, fold_ok=ffn.accepts_folded)
        stream.add(ffn.forward(h, ctx, lazy_output=True) if ffn.lazy_output else ffn.forward(h, ctx))


register_part("layer", "pre_norm", PreNormLayer)
