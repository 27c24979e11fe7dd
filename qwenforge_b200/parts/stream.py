"""Parts that work on the residual stream, or on a sublayer's input, between the blocks.

`embedding_mix` (role "stream"): the stream is replaced by a product over itself and the embedding's output side by side,
    x <- M [x ; e],  M [W, 2W], x's half first.
A schedule entry that names it in `enter` has the whole stream pass through it right before its block runs: the start of
every pass over a run of layers that repeats, for instance. The product's result is the new float32 stream.

`token_shift` (role "mixer_input"): what a mixer reads is drawn towards the previous token's,
    u_t = h_t + (h_(t-1) - h_t) * s,  element by element, h before a sequence's first token being zero.
The previous h (as it was before this replacement) is part of a sequence's state: one float32 row per sequence and
schedule entry. Computed as the two-tap convolution s * h_(t-1) + (1 - s) * h_t over each sequence's tokens, float32 inside.
"""
from __future__ import annotations

import torch

from .. import ops
from ..cache import StateNeed
from .base import Part, Pending, PendingPair, TensorSpec
from .registry import register_part


class EmbeddingMix(Part):
    """params: width. tensors: weight [width, 2 * width]."""

    def __init__(self, spec):
        super().__init__(spec)
        self.width = int(self.params["width"])
        self.weight = None

    def tensor_specs(self):
        return [TensorSpec(self.file_name("weight"), (self.width, 2 * self.width))]

    def kernel_libraries(self, dtype):
        return {"norm"} | ({"gemm_f32"} if dtype == torch.float32 else {"skinny_gemm"})

    def bind(self, tensors, dtype, device):
        self.weight = tensors[self.file_name("weight")]

    def step_weights(self):
        return [self.weight]

    def forward(self, hidden, delta, first, ctx):
        """The new stream. `delta`: what is still pending for `hidden` (None, a tensor, or a pair); `first`: the
        embedding's output [T, W] float32."""
        if isinstance(delta, Pending) and not isinstance(delta, PendingPair):
            delta.add_to(hidden)
            delta = None
        a, b = (delta.a, delta.b) if isinstance(delta, PendingPair) else (delta, None)
        both = torch.empty((hidden.shape[0], 2 * self.width), dtype=self.weight.dtype, device=hidden.device)
        ops.stream_pair(hidden, a, b, first, both)
        return ops.linear_rows(both, self.weight, out_dtype=torch.float32)


class TokenShift(Part):
    """params: width. tensors: weight [width] (s above)."""

    def __init__(self, spec):
        super().__init__(spec)
        self.width = int(self.params["width"])
        self.taps = None

    def tensor_specs(self):
        return [TensorSpec(self.file_name("weight"), (self.width,), init="fraction", keep="float32")]

    def kernel_libraries(self, dtype):
        return {"recurrent"}

    def cache_need(self):
        return StateNeed((self.width,), torch.float32)

    def bind(self, tensors, dtype, device):
        s = tensors[self.file_name("weight")].to(torch.float32)
        self.taps = torch.stack((s, 1.0 - s), dim=1).contiguous()     # [W, 2]: the older input first

    def step_weights(self):
        return [self.taps]

    def rides_on_norm(self, n_rows: int, ctx, site):
        """What a norm kernel that takes a shift needs to do this part's work itself, in a step of one token per sequence
        (else None): the taps, the step's slots, the kept rows."""
        if not (ctx.is_decode and n_rows == ctx.n_seqs):
            return None
        return self.taps, ctx.slots, site.storage

    def forward(self, h: torch.Tensor, ctx, site) -> torch.Tensor:
        out = torch.empty_like(h)
        ops.causal_conv(h, self.taps, None, ctx.cu_q, ctx.tok_seq, ctx.slots, site.storage, 0, out,
                        single=ctx.is_decode and h.shape[0] == ctx.n_seqs)
        return out


register_part("stream", "embedding_mix", EmbeddingMix)
register_part("mixer_input", "token_shift", TokenShift)
