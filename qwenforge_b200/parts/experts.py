"""A mixture of small SwiGLU experts chosen per token by a router.

  z = R h (float32)                         router logits
  s = sigmoid(z)  or  softmax(z)            scores (`score`)
  the `top` experts with the largest s      weights: their scores, divided by their sum with `renormalize`
  out = sum_e expert_e(w_e * h)             `weight_on` = "input": the weight multiplies what the expert reads
     or sum_e w_e * expert_e(h)             `weight_on` = "output"
  expert(v) = D_e (silu(G_e v) * (U_e v)),  no biases
(computed as silu(w_e (G_e h)) * (w_e (U_e h)) for a weight on the input: the same numbers, the scale applied to float32 sums)

Options, each a parameter of the spec:
  router_bias  z = R h + r, a float32 bias per expert, added before the choice
  gate         "clamped": expert(v) = D_e (g * sigmoid(alpha g) * (u + 1)) with g = min(G_e v, limit), u = clamp(U_e v, -limit, limit)
               (`limit`, `alpha`) instead of the SwiGLU; the weight is then on the output
  shared       one more expert of the same form with sizes of its own (`size`, `limit`) that every token gets, added to the
               chosen experts' sum; with `gated` it is multiplied by sigmoid(s . h), one number per token
  gate         "none": the experts have no gate, expert(v) = D_e act(U_e v) with `activation` one of the library's (the square
               of relu, say); tensors up.<e>, down.<e> only, and the shared expert likewise
  correction   a float32 number per expert that is added to the sigmoid score for the CHOICE only; the weights are the
               scores without it
  groups       (count, keep): the experts form `count` equal groups of neighbours, a group's score is the sum of its two
               largest choice scores, and only experts of the `keep` best groups can be chosen
(score "softmax" with `renormalize` is the softmax over the chosen logits alone.)

Routing, sorting by expert and the experts' products all stay on the device (`ops.moe_plan`, `ops.expert_linear`: one
launch per product for all experts, sized by what any routing can need), so the part is graph safe: a decode graph
replays it with other routings every step.
"""
from __future__ import annotations

import torch

from .. import ops
from .base import FeedForward, RowSum, TensorSpec, fork, join, runs_side_by_side
from .registry import register_part


class RoutedExperts(FeedForward):
    """params: hidden_size, expert_size, experts, top, score ("sigmoid" | "softmax"), renormalize, weight_on ("input" | "output").
    tensors: router [E, W], and per expert e: gate.<e> [F, W], up.<e> [F, W], down.<e> [W, F]."""

    def __init__(self, spec):
        super().__init__(spec)
        p = self.params
        self.hidden = int(p["hidden_size"])
        self.inter = int(p["expert_size"])
        self.n_experts = int(p["experts"])
        self.top = int(p["top"])
        self.score = str(p.get("score", "sigmoid"))
        self.renormalize = bool(p.get("renormalize", False))
        self.weight_on = str(p.get("weight_on", "output"))
        if self.score not in ("sigmoid", "softmax") or self.weight_on not in ("input", "output"):
            raise ValueError(f"routed_experts: score {self.score!r} / weight_on {self.weight_on!r} not understood")
        if not 1 <= self.top <= min(self.n_experts, 16):
            raise ValueError(f"routed_experts: top {self.top} of {self.n_experts} experts is not supported (1..16)")
        self.router_bias = bool(p.get("router_bias", False))
        self.gate = str(p.get("gate", "swiglu"))
        self.limit, self.alpha = float(p.get("limit") or 0.0), float(p.get("alpha") or 0.0)
        if self.gate not in ("swiglu", "clamped", "none") or (self.gate == "clamped" and (self.weight_on != "output" or self.limit <= 0)):
            raise ValueError("routed_experts: gate is 'swiglu', 'clamped' or 'none'; the clamped gate takes a positive limit and the weight on the output")
        self.activation = str(p.get("activation") or "relu2")
        if self.gate == "none" and (self.weight_on != "output" or self.activation not in ops.ACTIVATIONS):
            raise ValueError("routed_experts: experts without a gate take one of the library's activations and the weight on the output")
        self.corrected = bool(p.get("correction", False))
        self.groups = tuple(int(g) for g in p["groups"]) if p.get("groups") else None
        if (self.corrected or self.groups) and self.score != "sigmoid":
            raise ValueError("routed_experts: a correction of the choice and groups of experts go with sigmoid scores")
        if self.groups and (not 1 <= self.groups[1] <= self.groups[0] <= 64 or self.n_experts % self.groups[0]
                            or self.groups[1] * (self.n_experts // self.groups[0]) < self.top):
            raise ValueError(f"routed_experts: {self.groups[1]} of {self.groups[0]} groups over {self.n_experts} experts cannot "
                             f"yield {self.top} choices (up to 64 equal groups)")
        self.correction = None
        self.shared = dict(p["shared"]) if p.get("shared") else None
        self.router = self.gate_up = self.down = self.bias = None
        self.shared_gate_up = self.shared_down = self.shared_logit = None
        # what a block that sums rows inside its next norm kernel may call instead of `forward`: only where the chosen
        # experts' rows are the whole output
        self.forward_rows = self._routed_rows if self.shared is None else None

    def tensor_specs(self):
        specs = [TensorSpec(self.file_name("router"), (self.n_experts, self.hidden))]
        for e in range(self.n_experts):
            if self.gate != "none":
                specs.append(TensorSpec(self.file_name(f"gate.{e}"), (self.inter, self.hidden)))
            specs += [TensorSpec(self.file_name(f"up.{e}"), (self.inter, self.hidden)),
                      TensorSpec(self.file_name(f"down.{e}"), (self.hidden, self.inter))]
        if self.corrected:
            specs.append(TensorSpec(self.file_name("correction"), (self.n_experts,), init="bias", keep="float32"))
        if self.router_bias:
            specs.append(TensorSpec(self.file_name("router_bias"), (self.n_experts,), init="logit", keep="float32"))
        if self.shared is not None:
            size = int(self.shared["size"])
            if self.gate != "none":
                specs.append(TensorSpec(self.file_name("shared_gate"), (size, self.hidden)))
            specs += [TensorSpec(self.file_name("shared_up"), (size, self.hidden)), TensorSpec(self.file_name("shared_down"), (self.hidden, size))]
            if self.shared.get("gated"):
                specs.append(TensorSpec(self.file_name("shared_logit"), (1, self.hidden)))
        return specs

    def kernel_libraries(self, dtype):
        return {"activation", "moe", "grouped_gemm"} | ({"gemm_f32"} if dtype == torch.float32 else {"tc_gemm"})

    def bind(self, tensors, dtype, device):
        t = lambda logical: tensors[self.file_name(logical)]
        self.router = t("router")
        if self.corrected:
            self.correction = t("correction").to(torch.float32).contiguous()
        if self.gate == "none":   # (`gate_up` holds the one first product's weights)
            self.gate_up = torch.stack([t(f"up.{e}") for e in range(self.n_experts)]).contiguous()
        else:
            self.gate_up = torch.stack([torch.cat((t(f"gate.{e}"), t(f"up.{e}")), dim=0) for e in range(self.n_experts)]).contiguous()
        self.down = torch.stack([t(f"down.{e}") for e in range(self.n_experts)]).contiguous()
        if self.router_bias:
            self.bias = t("router_bias").to(torch.float32).contiguous()
        if self.shared is not None:
            self.shared_gate_up = t("shared_up") if self.gate == "none" else torch.cat((t("shared_gate"), t("shared_up")), dim=0).contiguous()
            self.shared_down = t("shared_down")
            if self.shared.get("gated"):
                self.shared_logit = t("shared_logit")

    def step_weights(self):
        return [w for w in (self.router, self.gate_up, self.down, self.bias, self.correction, self.shared_gate_up, self.shared_down,
                            self.shared_logit) if w is not None]

    def _shared_rows(self, x):
        """The expert that every token gets: [T, W], not yet gated."""
        act = torch.empty((x.shape[0], int(self.shared["size"])), dtype=x.dtype, device=x.device)
        if self.gate == "none":
            ops.bias_act(ops.linear_rows(x, self.shared_gate_up), None, self.activation, act)
        elif self.gate == "clamped":
            limit = float(self.shared.get("limit") or self.limit)
            if not ops.gated_rows(x, self.shared_gate_up, act, clamp=(limit, self.alpha)):   # few rows: the gate in the product
                ops.clamped_glu(ops.linear_rows(x, self.shared_gate_up), limit, self.alpha, act)
        else:
            ops.swiglu(ops.linear_rows(x, self.shared_gate_up), act)
        return ops.linear_rows(act, self.shared_down)

    def forward(self, x, ctx):
        out = torch.empty_like(x)
        extra = None
        if self.shared is not None and runs_side_by_side(x):
            # a step of few rows: the shared expert's chain of kernels on a stream of its own beside the routed experts'
            main, side = fork(x)
            with torch.cuda.stream(side):
                extra = self._shared_rows(x)
            r = self._routed_rows(x, ctx)
            join(main, side, extra)
        else:
            r = self._routed_rows(x, ctx)
            if self.shared is not None:   # the expert that every token gets rides on the kernel that sums the chosen ones
                extra = self._shared_rows(x)
        # (the shared expert's gate, one logit per token, is formed inside the kernel that sums)
        ops.moe_combine(r.rows, self._plan, out, r.row_weight is not None, extra, None, x if self.shared_logit is not None else None,
                        self.shared_logit.view(-1) if self.shared_logit is not None else None)
        return out

    def _routed_rows(self, x, ctx) -> RowSum:
        """The chosen experts' output rows, `top` per token and not yet summed (see `RowSum`)."""
        # float32 logits from the rows as the experts see them (their bfloat16 rounding on the 16-bit path: products of
        # bfloat16 numbers are exact in float32, and the sums are float32)
        n = x.shape[0]
        # (the large tile only where both products' operands allow it)
        tile_rows = min(ops.moe_tile_rows(n, self.n_experts, self.top, self.gate_up), ops.moe_tile_rows(n, self.n_experts, self.top, self.down))
        soft, renorm = self.score == "softmax", self.renormalize
        choice = {"correction": self.correction, "groups": self.groups} if (self.corrected or self.groups) else {}
        if n * self.n_experts <= ops.MOE_FUSED_ROUTER_MAX:
            plan = ops.moe_plan(None, self.top, soft, renorm, tile_rows, x=x, router=self.router, bias=self.bias, **choice)   # few tokens: one launch
        else:
            plan = ops.moe_plan(ops.linear(x, self.router, out_dtype=torch.float32), self.top, soft, renorm, tile_rows, bias=self.bias,
                                **choice)
        self._plan = plan
        if self.gate == "none":
            act = torch.empty((plan.pairs, self.inter), dtype=x.dtype, device=x.device)
            rows = torch.empty((plan.pairs, self.hidden), dtype=x.dtype, device=x.device)
            if tile_rows == ops.kernels.GROUP_LARGE_TILE_ROWS and ops.tc_gemm_grouped_takes(rows, self.gate_up, plan) \
                    and ops.tc_gemm_grouped_takes(act, self.down, plan):
                # long steps: both products on the tcgen05 tensor cores (their tiled copies want the sorted rows in memory)
                ops.moe_gather(x, plan, rows, False)
                up = torch.empty_like(act)
                ops.tc_gemm_grouped(ops.TC_PLAIN, rows, self.gate_up, plan, up, None, ctx.err)
                ops.bias_act(up, None, self.activation, act)
                y = torch.empty_like(rows)
                ops.tc_gemm_grouped(ops.TC_PLAIN, act, self.down, plan, y, None, ctx.err)
                return RowSum(y, plan.dest, self.top, plan.sorted_weight)
            # the rows are read through the plan's row map; the activation in the first product's epilogue
            ops.expert_linear(x, self.gate_up, plan, act, gather=True, activation=self.activation)
            ops.expert_linear(act, self.down, plan, rows)
            return RowSum(rows, plan.dest, self.top, plan.sorted_weight)
        if self.gate == "clamped":
            act = torch.empty((plan.pairs, self.inter), dtype=x.dtype, device=x.device)
            rows = torch.empty((plan.pairs, self.hidden), dtype=x.dtype, device=x.device)
            if tile_rows == ops.kernels.GROUP_LARGE_TILE_ROWS and ops.tc_gemm_grouped_takes(rows, self.gate_up, plan, ops.TC_SWIGLU) \
                    and ops.tc_gemm_grouped_takes(act, self.down, plan):
                # long steps: both products on the tcgen05 tensor cores, the clamped gate in the first one's epilogue
                ops.moe_gather(x, plan, rows, False)
                ops.tc_gemm_grouped(ops.TC_SWIGLU, rows, self.gate_up, plan, act, None, ctx.err, clamp=(self.limit, self.alpha))
                y = torch.empty_like(rows)
                ops.tc_gemm_grouped(ops.TC_PLAIN, act, self.down, plan, y, None, ctx.err)
                return RowSum(y, plan.dest, self.top, plan.sorted_weight)
            # otherwise the rows are read through the plan's row map: the clamped gate in the product's epilogue where the small
            # tensor-core tile takes the operands, else both halves in one product and the gate behind it
            if self.limit > 0 and ops.expert_gate_takes(x, self.gate_up, plan):
                ops.expert_gate_up(x, self.gate_up, plan, act, None, gather=True, clamp=(self.limit, self.alpha))
            else:
                gate_up = torch.empty((plan.pairs, 2 * self.inter), dtype=x.dtype, device=x.device)
                ops.expert_linear(x, self.gate_up, plan, gate_up, gather=True)
                ops.clamped_glu(gate_up, self.limit, self.alpha, act)
            ops.expert_linear(act, self.down, plan, rows)
            return RowSum(rows, plan.dest, self.top, plan.sorted_weight)
        # A weight on the expert's input moves behind its first product (G (w h) = w (G h), and the same for U), where it
        # meets float32 sums.
        on_input = self.weight_on == "input"
        act = torch.empty((plan.pairs, self.inter), dtype=x.dtype, device=x.device)
        rows = torch.empty((plan.pairs, self.hidden), dtype=x.dtype, device=x.device)
        if tile_rows == ops.kernels.GROUP_LARGE_TILE_ROWS and ops.tc_gemm_grouped_takes(rows, self.gate_up, plan, ops.TC_SWIGLU) \
                and ops.tc_gemm_grouped_takes(act, self.down, plan):
            # long steps: both products on the tcgen05 tensor cores, the gate in the first one's epilogue (its tiled copies
            # want the sorted rows in memory, so they are gathered first)
            ops.moe_gather(x, plan, rows, False)
            ops.tc_gemm_grouped(ops.TC_SWIGLU, rows, self.gate_up, plan, act, plan.sorted_weight if on_input else None, ctx.err)
            y = torch.empty_like(rows)
            ops.tc_gemm_grouped(ops.TC_PLAIN, act, self.down, plan, y, None, ctx.err)
            return RowSum(y, plan.dest, self.top, None if on_input else plan.sorted_weight)
        # otherwise the sorted rows are read through the plan's row map and never stored
        if ops.expert_gate_takes(x, self.gate_up, plan):   # the gate in the product's epilogue
            ops.expert_gate_up(x, self.gate_up, plan, act, plan.sorted_weight if on_input else None, gather=True)
        else:
            gate_up = torch.empty((plan.pairs, 2 * self.inter), dtype=x.dtype, device=x.device)
            ops.expert_linear(x, self.gate_up, plan, gate_up, gather=True)
            if on_input:
                ops.scaled_swiglu(gate_up, plan.sorted_weight, act)
            else:
                ops.swiglu(gate_up, act)
        ops.expert_linear(act, self.down, plan, rows)
        return RowSum(rows, plan.dest, self.top, None if on_input else plan.sorted_weight)


register_part("feed_forward", "routed_experts", RoutedExperts)
