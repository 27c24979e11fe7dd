"""Two mixers side by side: both read the same input, and the layer's output is a weighted sum of theirs,
    out = left_scale * left(h) + right_scale * right(h).
Each keeps what it needs per sequence under its own name (`left`, `right`) in the schedule entry's bundle. The two outputs
are not summed here: they go to the block as a pair with a factor each, and the kernel of the norm that reads the stream
next adds them in float32.

In a step of few rows on a GPU the two sides run on two streams: the right side forks off the step's stream at the mixer's
input and joins it again before the block goes on. Such a step is a chain of short dependent kernels, and two chains side by
side are as long as the longer one (measured at Qwen2.5-0.5B sizes, batch 8: 2.29 -> 2.12 ms per decode step; `fork` and
`join` in `parts/base.py`). A capture of the step's stream takes the fork and the join with it. Long steps run one side after the other: there both sides' products
fill the GPU, and a recurrent scan, which holds a few dozen SMs and is bound by its own chain of instructions, only slows
down when another kernel's blocks share its SMs (a 2,048-token prompt: 8.88 ms on one stream, 9.0 on two, also with the left
side held back until the scan has started)."""
from __future__ import annotations

import torch

from ..cache import BundleNeed
from .base import Mixer, PendingScaled, fork, join, runs_side_by_side
from .registry import build_part, register_part


class SideBySide(Mixer):
    """params: left, right (PartSpecs of role "mixer"), left_scale, right_scale."""

    scaled_outputs = True   # `forward` hands back a `PendingScaled`, which a block must know how to take
    concurrent = True       # on a GPU the right side runs on a stream of its own beside the left one

    def __init__(self, spec):
        super().__init__(spec)
        self.left = build_part("mixer", self.params["left"])
        self.right = build_part("mixer", self.params["right"])
        self.left_scale, self.right_scale = float(self.params["left_scale"]), float(self.params["right_scale"])
        for side in (self.left, self.right):
            if getattr(side, "scaled_outputs", False):
                raise ValueError("side_by_side: each side must be a mixer with one output")

    def sub_parts(self):
        return [self.left, self.right]

    def cache_need(self):
        needs = tuple((name, side.cache_need()) for name, side in (("left", self.left), ("right", self.right))
                      if side.cache_need() is not None)
        return BundleNeed(needs) if needs else None

    def forward(self, x, ctx, site, writes_cache):
        if not writes_cache:
            raise ValueError("side_by_side: two mixers with states of their own cannot read another entry's cache")
        pick = lambda name, side: site[name] if side.cache_need() is not None else None
        if not (self.concurrent and runs_side_by_side(x)):
            left = self.left.forward(x, ctx, pick("left", self.left), True)
            right = self.right.forward(x, ctx, pick("right", self.right), True)
            return PendingScaled(left, self.left_scale, right, self.right_scale)
        main, side = fork(x)             # the right side starts where the mixer's input is ready
        with torch.cuda.stream(side):
            right = self.right.forward(x, ctx, pick("right", self.right), True)
        left = self.left.forward(x, ctx, pick("left", self.left), True)
        join(main, side, right)          # whoever reads the pair next runs on the step's stream
        return PendingScaled(left, self.left_scale, right, self.right_scale)


register_part("mixer", "side_by_side", SideBySide)
