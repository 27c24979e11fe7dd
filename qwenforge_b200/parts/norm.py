"""RMSNorm: x * rsqrt(mean(x^2) + eps) * w, statistics in float32 (student_engine.py:530-535).

The residual stream is float32 in both precisions; the addition of the previous part's output
is fused into this kernel, so the stream is read once and written once per norm."""
from __future__ import annotations

from typing import Optional

import torch

from .. import ops
from .base import Norm, PendingScaled, TensorSpec
from .registry import register_part


class RmsNorm(Norm):
    """params: width, eps. tensors: weight [width]."""

    def __init__(self, spec):
        super().__init__(spec)
        self.width = int(self.params["width"])
        self.eps = float(self.params["eps"])
        self.weight = None

    def tensor_specs(self):
        return [TensorSpec(self.file_name("weight"), (self.width,), init="norm")]

    def kernel_libraries(self, dtype):
        return {"norm"}

    def bind(self, tensors, dtype, device):
        self.weight = tensors[self.file_name("weight")]

    def forward(self, hidden: torch.Tensor, delta) -> torch.Tensor:
        """delta: None, a tensor, or a `PendingScaled` (outputs that enter the stream under a factor each, added by this
        norm's kernel on its way)."""
        out = torch.empty(hidden.shape, dtype=self.weight.dtype, device=hidden.device)
        if isinstance(delta, PendingScaled):
            ops.add_rms_norm_scaled(hidden, delta.a, delta.scale_a, delta.b, delta.scale_b, self.weight, self.eps, out)
        else:
            ops.add_rms_norm(hidden, delta, self.weight, self.eps, out)
        return out

    def fused_rms(self):
        return self.weight, self.eps

    def step_weights(self):
        return [self.weight]


class DynamicTanh(Norm):
    """Dynamic Tanh in a norm's place: tanh(alpha * x) * w + b, element by element; no mean, no variance, no eps.
    params: width. tensors: weight [width], bias [width], alpha [] (a scalar, read once when the weights are bound).
    `forward` takes up to two pending outputs and adds their sum to the stream on its way (float32)."""
    takes_pair = True

    def __init__(self, spec):
        super().__init__(spec)
        self.width = int(self.params["width"])
        self.weight = self.bias = None
        self.alpha = 1.0

    def tensor_specs(self):
        return [TensorSpec(self.file_name("weight"), (self.width,), init="norm"),
                TensorSpec(self.file_name("bias"), (self.width,), init="bias"),
                TensorSpec(self.file_name("alpha"), (), init="norm", keep="float32")]

    def kernel_libraries(self, dtype):
        return {"norm"}

    def bind(self, tensors, dtype, device):
        self.weight = tensors[self.file_name("weight")]
        self.bias = tensors[self.file_name("bias")]
        self.alpha = float(tensors[self.file_name("alpha")].float().item())

    takes_shift = True

    def forward(self, hidden: torch.Tensor, delta: Optional[torch.Tensor], second: Optional[torch.Tensor] = None, shift=None):
        """shift: None, or (taps [W, 2] float32, slots [R], state [slots, >= W]) in a step of one token per sequence: the
        token shift behind this norm rides in its kernel, and the result is the pair (out, shifted)."""
        out = torch.empty(hidden.shape, dtype=self.weight.dtype, device=hidden.device)
        if shift is None:
            ops.add_dyt_norm(hidden, delta, second, self.weight, self.bias, self.alpha, out)
            return out
        shifted = torch.empty_like(out)
        ops.add_dyt_norm_shift(hidden, delta, second, self.weight, self.bias, self.alpha, out, shift[0], shift[1], shift[2], shifted)
        return out, shifted

    def step_weights(self):
        return [self.weight, self.bias]


register_part("norm", "rms_norm", RmsNorm)
register_part("norm", "dynamic_tanh", DynamicTanh)
