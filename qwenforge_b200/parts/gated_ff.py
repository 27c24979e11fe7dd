"""Feed-forwards with other gates than SwiGLU's.

`clamped_glu`: both halves of the gate/up product are clamped before they meet, the gate is x * sigmoid(alpha x) and
the linear half is shifted by one:
    g = min(G h, limit),  u = clamp(U h, -limit, limit),  out = D (g * sigmoid(alpha * g) * (u + 1))
Gate and up weights are concatenated by rows so that one product yields both halves; no biases.

`gated_mlp`: a gate of any of the library's activations, with optional biases on all three products:
    out = D (act(G h + bg) * (U h + bu)) + bd
The two first biases, the activation and the product of the halves are one kernel."""
from __future__ import annotations

import torch

from .. import ops
from .base import FeedForward, TensorSpec
from .registry import register_part


class ClampedGlu(FeedForward):
    """params: hidden_size, intermediate_size, limit, alpha. tensors: gate_weight [I, W], up_weight [I, W], down_weight [W, I]."""

    def __init__(self, spec):
        super().__init__(spec)
        self.hidden = int(self.params["hidden_size"])
        self.inter = int(self.params["intermediate_size"])
        self.limit = float(self.params["limit"])
        self.alpha = float(self.params["alpha"])
        self.gate_up_weight = self.down_weight = None

    def tensor_specs(self):
        return [
            TensorSpec(self.file_name("gate_weight"), (self.inter, self.hidden)),
            TensorSpec(self.file_name("up_weight"), (self.inter, self.hidden)),
            TensorSpec(self.file_name("down_weight"), (self.hidden, self.inter)),
        ]

    def kernel_libraries(self, dtype):
        return {"activation"} | ({"gemm_f32"} if dtype == torch.float32 else {"skinny_gemm"})

    def bind(self, tensors, dtype, device):
        self.gate_up_weight = torch.cat((tensors[self.file_name("gate_weight")], tensors[self.file_name("up_weight")]),
                                        dim=0).contiguous()
        self.down_weight = tensors[self.file_name("down_weight")]

    def step_weights(self):
        return [self.gate_up_weight, self.down_weight]

    def forward(self, x, ctx):
        act = torch.empty((x.shape[0], self.inter), dtype=x.dtype, device=x.device)
        ops.clamped_glu(ops.linear_rows(x, self.gate_up_weight), self.limit, self.alpha, act)
        return ops.linear_rows(act, self.down_weight)


class GatedMlp(FeedForward):
    """params: hidden_size, intermediate_size, activation, bias (bool). tensors: gate_weight [I, W], up_weight [I, W],
    down_weight [W, I] (+ gate_bias [I], up_bias [I], down_bias [W])."""

    def __init__(self, spec):
        super().__init__(spec)
        self.hidden = int(self.params["hidden_size"])
        self.inter = int(self.params["intermediate_size"])
        self.activation = str(self.params["activation"])
        self.bias = bool(self.params.get("bias", False))
        if self.activation not in ops.ACTIVATIONS:
            raise ValueError(f"gated_mlp: unknown activation {self.activation!r}; known: {', '.join(ops.ACTIVATIONS)}")
        self.gate_up_weight = self.down_weight = self.gate_up_bias = self.down_bias = None

    def tensor_specs(self):
        specs = [TensorSpec(self.file_name("gate_weight"), (self.inter, self.hidden)),
                 TensorSpec(self.file_name("up_weight"), (self.inter, self.hidden)),
                 TensorSpec(self.file_name("down_weight"), (self.hidden, self.inter))]
        if self.bias:
            specs += [TensorSpec(self.file_name("gate_bias"), (self.inter,), init="bias"),
                      TensorSpec(self.file_name("up_bias"), (self.inter,), init="bias"),
                      TensorSpec(self.file_name("down_bias"), (self.hidden,), init="bias")]
        return specs

    def kernel_libraries(self, dtype):
        return {"activation"} | ({"gemm_f32"} if dtype == torch.float32 else {"skinny_gemm"})

    def bind(self, tensors, dtype, device):
        t = lambda logical: tensors[self.file_name(logical)]
        self.gate_up_weight = torch.cat((t("gate_weight"), t("up_weight")), dim=0).contiguous()
        self.down_weight = t("down_weight")
        if self.bias:
            self.gate_up_bias = torch.cat((t("gate_bias"), t("up_bias"))).contiguous()
            self.down_bias = t("down_bias")

    def step_weights(self):
        return [t for t in (self.gate_up_weight, self.gate_up_bias, self.down_weight, self.down_bias) if t is not None]

    def forward(self, x, ctx):
        act = torch.empty((x.shape[0], self.inter), dtype=x.dtype, device=x.device)
        ops.bias_glu(ops.linear_rows(x, self.gate_up_weight), self.gate_up_bias, self.activation, act)
        if self.down_bias is None:
            return ops.linear_rows(act, self.down_weight)
        return ops.linear(act, self.down_weight, self.down_bias)


register_part("feed_forward", "clamped_glu", ClampedGlu)
register_part("feed_forward", "gated_mlp", GatedMlp)
