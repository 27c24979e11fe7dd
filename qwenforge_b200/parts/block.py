"""Arrangements of a layer's parts around the residual stream.

`pre_norm` (student_engine.py:696-731):  h += mixer(norm_1(h));  h += feed_forward(norm_2(h)).
The stream `hidden` is float32 and is updated in place; a part's output (`delta`) is added to it by
the *next* norm's kernel, so a block takes the pending delta of the layer before it and returns its own."""
from __future__ import annotations

import torch

from ..cache import BundleNeed
from .base import Norm, Part, PendingNormed, PendingPair, PendingScaled
from .registry import build_part, register_part


class PreNormBlock(Part):
    """Reads the layer spec's parts `mixer_norm`, `mixer` and, if the layer has a feed-forward, `feed_forward_norm` and
    `feed_forward`. With the layer spec's parameter `residual_mult` = m every sublayer's output enters the stream times m:
    h += m * mixer(norm_1(h));  h += m * feed_forward(norm_2(h))  (the product and the sum in float32, inside the next norm's
    kernel). A mixer may hand back two outputs under a factor each (`PendingScaled`); they go the same way."""

    accepts_pending = (PendingScaled,)

    def __init__(self, layer_spec):
        self.kind = "pre_norm"
        self.mixer_norm = build_part("norm", layer_spec.part("mixer_norm"))
        self.mixer = build_part("mixer", layer_spec.part("mixer"))
        self.feed_forward = self.feed_forward_norm = None
        if "feed_forward" in layer_spec.parts:
            self.feed_forward_norm = build_part("norm", layer_spec.part("feed_forward_norm"))
            self.feed_forward = build_part("feed_forward", layer_spec.part("feed_forward"))
        self.residual_mult = float(layer_spec.params.get("residual_mult", 1.0))

    def sub_parts(self):
        return [p for p in (self.mixer_norm, self.mixer, self.feed_forward_norm, self.feed_forward) if p is not None]

    def cache_need(self):
        return self.mixer.cache_need()

    def _forward_scaled(self, hidden, delta, ctx, site, writes_cache):
        """The layer with a residual multiplier, a mixer of two outputs, or no feed-forward: every output stays pending
        with its factor and is added, in float32, by the kernel of the norm that reads the stream next."""
        x = self.mixer_norm.forward(hidden, delta)
        delta = PendingScaled.of(self.mixer.forward(x, ctx, site, writes_cache), self.residual_mult)
        if self.feed_forward is None:
            return delta
        x = self.feed_forward_norm.forward(hidden, delta)
        return PendingScaled.of(self.feed_forward.forward(x, ctx), self.residual_mult)

    def forward(self, hidden, delta, ctx, site, writes_cache):
        if self.residual_mult != 1.0 or self.feed_forward is None or getattr(self.mixer, "scaled_outputs", False) \
                or isinstance(delta, PendingScaled):
            return self._forward_scaled(hidden, delta, ctx, site, writes_cache)
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


class SandwichBlock(Part):
    """Norms before AND after each sublayer:  h += post_1(mixer(norm_1(h)));  h += post_2(feed_forward(norm_2(h))).
    Reads the layer spec's parts `mixer_norm`, `mixer`, `mixer_post_norm` and, if the layer has a feed-forward,
    `feed_forward_norm`, `feed_forward`, `feed_forward_post_norm`. The norms after the sublayers must be plain RMS norms
    (`fused_rms`): each rides, with its addition into the stream, on the kernel of the norm that follows it
    (`ops.sandwich_norm`), the last one of a layer on the first norm of the next layer."""

    accepts_pending_normed = True

    def __init__(self, layer_spec):
        self.kind = "sandwich_norm"
        self.mixer_norm = build_part("norm", layer_spec.part("mixer_norm"))
        self.mixer = build_part("mixer", layer_spec.part("mixer"))
        self.mixer_post_norm = build_part("norm", layer_spec.part("mixer_post_norm"))
        self.feed_forward = self.feed_forward_norm = self.feed_forward_post_norm = None
        if "feed_forward" in layer_spec.parts:
            self.feed_forward_norm = build_part("norm", layer_spec.part("feed_forward_norm"))
            self.feed_forward = build_part("feed_forward", layer_spec.part("feed_forward"))
            self.feed_forward_post_norm = build_part("norm", layer_spec.part("feed_forward_post_norm"))
        for norm in (self.mixer_norm, self.mixer_post_norm, self.feed_forward_norm, self.feed_forward_post_norm):
            if norm is not None and type(norm).fused_rms is Norm.fused_rms:
                raise ValueError("sandwich_norm: the norms must be plain RMS norms")

    def sub_parts(self):
        return [p for p in (self.mixer_norm, self.mixer, self.mixer_post_norm, self.feed_forward_norm, self.feed_forward,
                            self.feed_forward_post_norm) if p is not None]

    def cache_need(self):
        return self.mixer.cache_need()

    def forward(self, hidden, delta, ctx, site, writes_cache):
        weight, eps = self.mixer_norm.fused_rms()
        if isinstance(delta, PendingNormed):
            x = torch.empty(hidden.shape, dtype=weight.dtype, device=hidden.device)
            delta.into(hidden, weight, eps, x)
        else:
            x = self.mixer_norm.forward(hidden, delta)
        y = self.mixer.forward(x, ctx, site, writes_cache)
        post = PendingNormed(y, *self.mixer_post_norm.fused_rms())
        if self.feed_forward is None:
            return post
        weight, eps = self.feed_forward_norm.fused_rms()
        x = torch.empty(hidden.shape, dtype=weight.dtype, device=hidden.device)
        post.into(hidden, weight, eps, x)
        # a feed-forward that leaves several rows per token hands them over unsummed: the next norm kernel adds them up
        run = getattr(self.feed_forward, "forward_rows", None) or self.feed_forward.forward
        return PendingNormed(run(x, ctx), *self.feed_forward_post_norm.fused_rms())


class ParallelBlock(Part):
    """One norm that both sublayers read:  h = norm(x);  x += mixer(in(h)) + feed_forward(h).
    Reads the layer spec's parts `norm`, `mixer` and, if the layer has them, `feed_forward` and `mixer_input` (a part of role
    "mixer_input" that filters what the mixer reads and may keep a state of its own per sequence, such as a token shift;
    the feed-forward reads h as it is). The two outputs stay pending as a pair: the next norm kernel of a block of this
    kind adds their sum to the float32 stream on its way."""

    accepts_pending = (PendingPair,)

    def __init__(self, layer_spec):
        self.kind = "parallel"
        self.norm = build_part("norm", layer_spec.part("norm"))
        self.mixer = build_part("mixer", layer_spec.part("mixer"))
        self.mixer_input = build_part("mixer_input", layer_spec.part("mixer_input")) if "mixer_input" in layer_spec.parts else None
        self.feed_forward = build_part("feed_forward", layer_spec.part("feed_forward")) if "feed_forward" in layer_spec.parts else None
        self.pair_norm = bool(getattr(self.norm, "takes_pair", False))   # its kernel adds two pending outputs on its way

    def sub_parts(self):
        return [p for p in (self.norm, self.mixer_input, self.mixer, self.feed_forward) if p is not None]

    def cache_need(self):
        need = self.mixer.cache_need()
        if self.mixer_input is None or self.mixer_input.cache_need() is None:
            return need
        return BundleNeed((("input", self.mixer_input.cache_need()), ("mixer", need)))

    def forward(self, hidden, delta, ctx, site, writes_cache):
        bundled = self.mixer_input is not None and self.mixer_input.cache_need() is not None
        if bundled and not writes_cache:
            raise ValueError("parallel: a layer whose mixer input keeps a state cannot read another entry's cache")
        # a mixer input that the norm's kernel can make on its way (single tokens): one launch for both
        rider = None
        if bundled and getattr(self.norm, "takes_shift", False) and hasattr(self.mixer_input, "rides_on_norm"):
            rider = self.mixer_input.rides_on_norm(hidden.shape[0], ctx, site["input"])
        extra = {} if rider is None else {"shift": rider}
        if isinstance(delta, PendingPair):
            if self.pair_norm:
                h = self.norm.forward(hidden, delta.a, delta.b, **extra)
            else:
                delta.add_to(hidden)
                h = self.norm.forward(hidden, None, **extra)
        else:
            h = self.norm.forward(hidden, delta, **extra)
        mixer_site, u = site, h
        if rider is not None:
            h, u = h
            mixer_site = site["mixer"]
        elif self.mixer_input is not None:
            u = self.mixer_input.forward(h, ctx, site["input"] if bundled else None)
            mixer_site = site["mixer"] if bundled else site
        mixed = self.mixer.forward(u, ctx, mixer_site, writes_cache)
        return PendingPair(mixed, self.feed_forward.forward(h, ctx) if self.feed_forward is not None else None)


register_part("block", "pre_norm", PreNormBlock)
register_part("block", "parallel", ParallelBlock)
register_part("block", "sandwich_norm", SandwichBlock)
