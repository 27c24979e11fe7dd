"""Recurrent mixers: a state of fixed size per sequence instead of keys and values per position.

Both kinds here keep, per head, a matrix S that every token decays and adds an outer product to, and read it with a
query:  S <- decay_t S + take_t k_t v_t^T,  y_t = S^T q_t  (`ops.outer_state_scan`, float32 inside). They differ in where
k, v, q and the two gates come from and in what follows the scan:

  matrix_memory (the mLSTM of xLSTM)
      q = Wq h / sqrt(dim), k = Wk h, v = Wv h in heads; exponential gates with a running maximum m (0 at a sequence's start):
      a = cap tanh((Wi h + bi) / cap),  f = logsigmoid(cap tanh((Wf h + bf) / cap)),  m' = max(f + m, a),
      decay = exp(f + m - m'), take = exp(a - m');  a vector n runs beside S with k alone;
      o = y / (max(|n . q|, exp(-m')) + floor);  out = Wo (unit_per_head(o) * w * sigmoid(Wg h))
  state_space (Mamba-2)
      [z | x | B | C | dt] = W_in h;  (x, B, C) <- silu(causal_conv(x, B, C) + b);  dt <- softplus(dt + dt_bias);
      decay = exp(-exp(A_log) dt), take = dt, k = B, q = C (shared by the heads of a group), v = x;
      y <- y + D x;  out = Wo (rms_in_parts(y * silu(z)) * w)

Two more kinds decay every ROW of S by a number of its own (a decay per head and key channel, `ops.outer_state_scan_rows`):

  time_mix (RWKV-style time mixing)
      with h' the token before (zeros at a sequence's start) each of r, k, v, g, w reads its own mix  h + (h' - h) mu_s;
      r, k, v = Wr ., Wk ., Wv . in heads of `dim`;  w = exp(-exp(W2 tanh(W1 .) + w0)) per head and channel;
      y_t = (S + diag(u) k_t v_t^T)^T r_t  with S as it was BEFORE the token (u: a learned bonus for the token itself);
      S <- diag(w_t) S + k_t v_t^T;   out = Wo (unit_per_head(y) * n * silu(Wg .))
  gated_linear_attention
      q = Wq h / sqrt(dim), k = Wk h, v = Wv h in heads;  a = sigmoid(A2 (A1 h) + b)^(1 / tau) per head and key channel;
      S <- diag(a_t) S + k_t v_t^T;  y_t = S^T q_t (AFTER the token);  out = Wo (rms_per_head(y; n) * silu(Wg h)),
      the norm's weight [vdim] shared by the heads

The state lives in the sequence cache as ONE float32 row per sequence and schedule entry (`StateNeed`), zeroed when a
sequence starts: [S | n | m] for the matrix memory, [S | the convolution's last taps - 1 inputs] for the state space,
[S | the last token's h] for the time mixing, [S] for the gated linear attention.
The gates' pre-activations are products with float32 results, and everything from there to the scan's output is
float32 in both precisions; the other projections and the convolution carry the activation dtype.
"""
from __future__ import annotations

import torch

from .. import ops
from ..cache import StateNeed
from .base import Mixer, TensorSpec, fork, join, runs_side_by_side
from .registry import register_part


class MatrixMemory(Mixer):
    """params: hidden_size, num_heads, head_dim, value_dim, gate_cap, eps, floor.
    tensors: q_weight, k_weight [H*dim, W], v_weight, g_weight [H*vdim, W], o_weight [W, H*vdim], norm [H*vdim],
    i_weight, f_weight [H, W], i_bias, f_bias [H]."""

    def __init__(self, spec):
        super().__init__(spec)
        p = self.params
        self.hidden, self.n_heads = int(p["hidden_size"]), int(p["num_heads"])
        self.dim, self.vdim = int(p["head_dim"]), int(p["value_dim"])
        self.cap, self.eps, self.floor = float(p["gate_cap"]), float(p["eps"]), float(p["floor"])
        if self.dim > ops.OUTER_STATE_MAX_DIM:
            raise ValueError(f"matrix_memory: head_dim {self.dim} > {ops.OUTER_STATE_MAX_DIM} is not supported by the scan kernel")
        h, d, v = self.n_heads, self.dim, self.vdim
        self.s_offset, self.n_offset, self.m_offset = 0, h * d * v, h * d * v + h * d
        self.state_floats = h * d * v + h * d + h
        self.proj_weight = self.gate_weight = self.gate_bias = self.norm = self.o_weight = None

    def tensor_specs(self):
        h, d, v, w = self.n_heads, self.dim, self.vdim, self.hidden
        f = self.file_name
        return [TensorSpec(f("q_weight"), (h * d, w)), TensorSpec(f("k_weight"), (h * d, w)), TensorSpec(f("v_weight"), (h * v, w)),
                TensorSpec(f("g_weight"), (h * v, w)), TensorSpec(f("o_weight"), (w, h * v)),
                TensorSpec(f("norm"), (h * v,), init="norm"), TensorSpec(f("i_weight"), (h, w)), TensorSpec(f("f_weight"), (h, w)),
                TensorSpec(f("i_bias"), (h,), init="bias", keep="float32"), TensorSpec(f("f_bias"), (h,), init="bias", keep="float32")]

    def kernel_libraries(self, dtype):
        return {"recurrent"} | ({"gemm_f32"} if dtype == torch.float32 else {"skinny_gemm"})

    def cache_need(self):
        return StateNeed((self.state_floats,), torch.float32)

    def bind(self, tensors, dtype, device):
        t = lambda logical: tensors[self.file_name(logical)]
        self.proj_weight = torch.cat((t("q_weight"), t("k_weight"), t("v_weight"), t("g_weight")), dim=0).contiguous()
        self.gate_weight = torch.cat((t("i_weight"), t("f_weight")), dim=0).contiguous()
        self.gate_bias = torch.cat((t("i_bias"), t("f_bias"))).to(torch.float32).contiguous()
        self.norm, self.o_weight = t("norm"), t("o_weight")

    def step_weights(self):
        return [self.proj_weight, self.gate_weight, self.gate_bias, self.norm, self.o_weight]

    def forward(self, x, ctx, site, writes_cache):
        if not writes_cache:
            raise ValueError("matrix_memory: a recurrent state cannot be read from another schedule entry")
        n, h, d, v = x.shape[0], self.n_heads, self.dim, self.vdim
        f32 = dict(dtype=torch.float32, device=x.device)
        proj = ops.linear_rows(x, self.proj_weight)                                   # [T, q | k | v | g]
        pre = ops.linear_rows(x, self.gate_weight, out_dtype=torch.float32)           # [T, i | f], float32 sums
        decay, take, floor = (torch.empty((n, h), **f32) for _ in range(3))
        ops.stabilized_gates(pre, self.gate_bias, self.cap, ctx.cu_q, ctx.slots, site.storage, self.m_offset, h, decay, take, floor)
        y, nq = torch.empty((n, h * v), **f32), torch.empty((n, h), **f32)
        ops.outer_state_scan(proj[:, :h * d], proj[:, h * d:2 * h * d], proj[:, 2 * h * d:2 * h * d + h * v], decay, take,
                             ctx.cu_q, ctx.slots, site.storage, self.s_offset, self.n_offset, h, h, d, v, d ** -0.5, y, nq)
        out = torch.empty((n, h * v), dtype=x.dtype, device=x.device)
        ops.gated_group_norm(y, proj[:, 2 * h * d + h * v:], self.norm, self.eps, out, h, h, "sigmoid", False,
                             nq=nq, floor=floor, floor_add=self.floor)
        return ops.linear_rows(out, self.o_weight)


class StateSpace(Mixer):
    """params: hidden_size, num_heads, value_dim, state_size, groups, conv_taps, norm_parts, eps.
    tensors: in_weight [2*inner + 2*G*N + H, W], conv_weight [inner + 2*G*N, taps], conv_bias, dt_bias [H], rate_log [H],
    skip [H], norm [inner], o_weight [W, inner]."""

    def __init__(self, spec):
        super().__init__(spec)
        p = self.params
        self.hidden, self.n_heads, self.vdim = int(p["hidden_size"]), int(p["num_heads"]), int(p["value_dim"])
        self.n_state, self.groups, self.taps = int(p["state_size"]), int(p["groups"]), int(p["conv_taps"])
        self.norm_parts, self.eps = int(p["norm_parts"]), float(p["eps"])
        self.inner = self.n_heads * self.vdim
        self.channels = self.inner + 2 * self.groups * self.n_state
        if self.n_heads % self.groups or self.inner % self.norm_parts:
            raise ValueError("state_space: the groups must divide the heads and the norm's parts the inner width")
        if self.n_state > ops.OUTER_STATE_MAX_DIM or not 1 <= self.taps <= ops.CONV_MAX_TAPS:
            raise ValueError(f"state_space: state_size up to {ops.OUTER_STATE_MAX_DIM} and 1 to {ops.CONV_MAX_TAPS} taps are supported")
        self.s_offset, self.conv_offset = 0, self.n_heads * self.n_state * self.vdim
        self.state_floats = self.conv_offset + (self.taps - 1) * self.channels
        self.main_weight = self.dt_weight = self.conv_weight = self.conv_bias = self.dt_bias = self.rate_log = self.skip = None
        self.norm = self.o_weight = None

    def tensor_specs(self):
        f, h = self.file_name, self.n_heads
        return [TensorSpec(f("in_weight"), (self.inner + self.channels + h, self.hidden)),
                TensorSpec(f("conv_weight"), (self.channels, self.taps), keep="float32"),
                TensorSpec(f("conv_bias"), (self.channels,), init="bias", keep="float32"),
                TensorSpec(f("dt_bias"), (h,), init="bias", keep="float32"), TensorSpec(f("rate_log"), (h,), init="bias", keep="float32"),
                TensorSpec(f("skip"), (h,), init="norm", keep="float32"), TensorSpec(f("norm"), (self.inner,), init="norm"),
                TensorSpec(f("o_weight"), (self.hidden, self.inner))]

    def kernel_libraries(self, dtype):
        return {"recurrent"} | ({"gemm_f32"} if dtype == torch.float32 else {"skinny_gemm"})

    def cache_need(self):
        return StateNeed((self.state_floats,), torch.float32)

    def bind(self, tensors, dtype, device):
        t = lambda logical: tensors[self.file_name(logical)]
        w = t("in_weight")
        self.main_weight = w[:self.inner + self.channels].contiguous()    # z | x | B | C
        self.dt_weight = w[self.inner + self.channels:].contiguous()      # dt: its sums stay float32
        self.conv_weight, self.conv_bias = t("conv_weight").float().contiguous(), t("conv_bias").float().contiguous()
        self.dt_bias, self.rate_log, self.skip = (t(k).float().contiguous() for k in ("dt_bias", "rate_log", "skip"))
        self.norm, self.o_weight = t("norm"), t("o_weight")

    def step_weights(self):
        return [self.main_weight, self.dt_weight, self.conv_weight, self.conv_bias, self.dt_bias, self.rate_log, self.skip,
                self.norm, self.o_weight]

    def forward(self, x, ctx, site, writes_cache):
        if not writes_cache:
            raise ValueError("state_space: a recurrent state cannot be read from another schedule entry")
        n, h, v, s, g = x.shape[0], self.n_heads, self.vdim, self.n_state, self.groups
        f32 = dict(dtype=torch.float32, device=x.device)
        main = ops.linear_rows(x, self.main_weight)                                   # [T, z | x | B | C]
        dt_pre = ops.linear_rows(x, self.dt_weight, out_dtype=torch.float32)          # [T, H], float32 sums
        xbc = torch.empty((n, self.channels), dtype=x.dtype, device=x.device)
        ops.causal_conv_silu(main[:, self.inner:], self.conv_weight, self.conv_bias, ctx.cu_q, ctx.tok_seq, ctx.slots,
                             site.storage, self.conv_offset, xbc, single=ctx.is_decode and n == ctx.n_seqs)
        decay, take = torch.empty((n, h), **f32), torch.empty((n, h), **f32)
        ops.decay_gates(dt_pre, self.dt_bias, self.rate_log, decay, take)
        y = torch.empty((n, self.inner), **f32)
        xs, b, c = xbc[:, :self.inner], xbc[:, self.inner:self.inner + g * s], xbc[:, self.inner + g * s:]
        ops.outer_state_scan(c, b, xs, decay, take, ctx.cu_q, ctx.slots, site.storage, self.s_offset, -1, h, g, s, v, 1.0, y, None)
        out = torch.empty((n, self.inner), dtype=x.dtype, device=x.device)
        ops.gated_group_norm(y, main[:, :self.inner], self.norm, self.eps, out, self.norm_parts, h, "silu", True,
                             skip=self.skip, skip_x=xs)
        return ops.linear_rows(out, self.o_weight)


def _rank_of(params, key="rank") -> int:
    """The rank of a low-rank pair of matrices: named by the spec, or -1 where only the weight files give it."""
    return int(params[key]) if params.get(key) else -1


def _low_rank(x, first, second, activation):
    """second act(first x) with float32 sums out: two products and the activation between them; the middle carries the
    activation dtype. (One kernel for both products of a step of few rows was measured at 29 and 48 microseconds against 13
    for the three launches at widths 896 and 2,048: the weight streamer has all of a product's weight bytes on their way at
    once, and a kernel that walks the rank row by row pays a round trip to memory per group of rows.)"""
    low = ops.linear_rows(x, first)
    if activation is not None:
        bent = torch.empty_like(low)
        ops.bias_act(low, None, activation, bent)
        low = bent
    return ops.linear_rows(low, second, out_dtype=torch.float32)


class TimeMix(Mixer):
    """params: hidden_size, num_heads, head_dim, eps, and optionally rank (of the decay's low-rank pair; read from the
    tensors where absent).
    tensors: mu_r, mu_k, mu_v, mu_g, mu_w [W]; r_weight, k_weight, v_weight, g_weight [H*dim, W]; w1 [rank, W], w2 [H*dim, rank],
    w0 [H*dim]; bonus [H, dim]; norm [H*dim]; o_weight [W, H*dim]."""

    MIXES = ("r", "k", "v", "g", "w")

    def __init__(self, spec):
        super().__init__(spec)
        p = self.params
        self.hidden, self.n_heads, self.dim = int(p["hidden_size"]), int(p["num_heads"]), int(p["head_dim"])
        self.eps, self.rank = float(p["eps"]), _rank_of(p)
        if self.dim > ops.OUTER_STATE_MAX_DIM:
            raise ValueError(f"time_mix: head_dim {self.dim} > {ops.OUTER_STATE_MAX_DIM} is not supported by the scan kernel")
        self.inner = self.n_heads * self.dim
        self.s_offset, self.h_offset = 0, self.n_heads * self.dim * self.dim
        self.state_floats = self.h_offset + self.hidden
        self.mu = self.proj_weight = self.w1 = self.w2 = self.w0 = self.bonus = self.norm = self.o_weight = None

    def tensor_specs(self):
        f, c, w = self.file_name, self.inner, self.hidden
        specs = [TensorSpec(f("mu_" + s), (w,), init="fraction", keep="float32") for s in self.MIXES]
        specs += [TensorSpec(f(s + "_weight"), (c, w)) for s in "rkvg"]
        return specs + [TensorSpec(f("w1"), (self.rank, w)), TensorSpec(f("w2"), (c, self.rank), init="low_rank"),
                        TensorSpec(f("w0"), (c,), init="rate", keep="float32"),
                        TensorSpec(f("bonus"), (self.n_heads, self.dim), init="logit", keep="float32"),
                        TensorSpec(f("norm"), (c,), init="norm"), TensorSpec(f("o_weight"), (w, c))]

    def kernel_libraries(self, dtype):
        return {"recurrent", "activation", "grouped_gemm"} | ({"gemm_f32"} if dtype == torch.float32 else {"skinny_gemm"})

    def cache_need(self):
        return StateNeed((self.state_floats,), torch.float32)

    def bind(self, tensors, dtype, device):
        t = lambda logical: tensors[self.file_name(logical)]
        self.mu = torch.stack([t("mu_" + s).to(torch.float32) for s in self.MIXES]).contiguous()       # [5, W]: r, k, v, g, w
        self.proj_weight = torch.stack([t(s + "_weight") for s in "rkvg"]).contiguous()                  # [4, H*dim, W]
        self.w1, self.w2 = t("w1").contiguous(), t("w2").contiguous()
        self.rank = int(self.w1.shape[0])
        self.w0, self.bonus = t("w0").to(torch.float32).contiguous(), t("bonus").to(torch.float32).contiguous()
        self.norm, self.o_weight = t("norm"), t("o_weight")

    def step_weights(self):
        return [self.mu, self.proj_weight, self.w1, self.w2, self.w0, self.bonus, self.norm, self.o_weight]

    def forward(self, x, ctx, site, writes_cache):
        if not writes_cache:
            raise ValueError("time_mix: a recurrent state cannot be read from another schedule entry")
        n, w, h, d, c = x.shape[0], self.hidden, self.n_heads, self.dim, self.inner
        f32 = dict(dtype=torch.float32, device=x.device)
        mixes = torch.empty((n, 5 * w), dtype=x.dtype, device=x.device)                 # [T, r | k | v | g | w], each W wide
        ops.shift_mix(x, self.mu, ctx.cu_q, ctx.tok_seq, ctx.slots, site.storage, self.h_offset, mixes,
                      single=ctx.is_decode and n == ctx.n_seqs)
        proj = torch.empty((n, 4 * c), dtype=x.dtype, device=x.device)                  # [T, r | k | v | g]
        if n > ops.WIDE_MAX_ROWS:   # long steps: a library product per mix
            for i in range(4):
                ops.linear(mixes[:, i * w:(i + 1) * w], self.proj_weight[i], out=proj[:, i * c:(i + 1) * c])
            pre = _low_rank(mixes[:, 4 * w:], self.w1, self.w2, "tanh")                  # float32 sums
        elif runs_side_by_side(mixes):   # few rows: the decays' chain of three kernels beside the four projections' one launch
            main, side = fork(mixes)
            with torch.cuda.stream(side):
                pre = _low_rank(mixes[:, 4 * w:], self.w1, self.w2, "tanh")
            ops.head_linear(mixes[:, :4 * w], self.proj_weight, proj)
            join(main, side, pre)
        else:
            ops.head_linear(mixes[:, :4 * w], self.proj_weight, proj)
            pre = _low_rank(mixes[:, 4 * w:], self.w1, self.w2, "tanh")
        y = torch.empty((n, c), **f32)   # (the scan forms the decays exp(-exp(pre + w0)) on its way in)
        ops.outer_state_scan_rows(proj[:, :c], proj[:, c:2 * c], proj[:, 2 * c:3 * c], pre, ctx.cu_q, ctx.slots, site.storage,
                                  self.s_offset, h, d, d, 1.0, y, bonus=self.bonus, decay_from=("double_exp", self.w0, 1.0))
        out = torch.empty((n, c), dtype=x.dtype, device=x.device)
        ops.gated_group_norm(y, proj[:, 3 * c:], self.norm, self.eps, out, h, h, "silu", False)
        return ops.linear_rows(out, self.o_weight)


class GatedLinearAttention(Mixer):
    """params: hidden_size, num_heads, head_dim, value_dim, tau, eps, and optionally rank (of the decay's low-rank pair).
    tensors: q_weight, k_weight [H*dim, W], v_weight, g_weight [H*vdim, W], o_weight [W, H*vdim], norm [vdim],
    a1 [rank, W], a2 [H*dim, rank], a2_bias [H*dim]."""

    def __init__(self, spec):
        super().__init__(spec)
        p = self.params
        self.hidden, self.n_heads = int(p["hidden_size"]), int(p["num_heads"])
        self.dim, self.vdim = int(p["head_dim"]), int(p["value_dim"])
        self.tau, self.eps, self.rank = float(p["tau"]), float(p["eps"]), _rank_of(p)
        if self.dim > ops.OUTER_STATE_MAX_DIM or self.tau <= 0:
            raise ValueError(f"gated_linear_attention: head_dim up to {ops.OUTER_STATE_MAX_DIM} and a positive tau are supported")
        self.state_floats = self.n_heads * self.dim * self.vdim
        self.proj_weight = self.a1 = self.a2 = self.a2_bias = self.norm = self.o_weight = None

    def tensor_specs(self):
        f, h, d, v, w = self.file_name, self.n_heads, self.dim, self.vdim, self.hidden
        return [TensorSpec(f("q_weight"), (h * d, w)), TensorSpec(f("k_weight"), (h * d, w)), TensorSpec(f("v_weight"), (h * v, w)),
                TensorSpec(f("g_weight"), (h * v, w)), TensorSpec(f("o_weight"), (w, h * v)), TensorSpec(f("norm"), (v,), init="norm"),
                TensorSpec(f("a1"), (self.rank, w)), TensorSpec(f("a2"), (h * d, self.rank), init="low_rank"),
                TensorSpec(f("a2_bias"), (h * d,), init="logit", keep="float32")]

    def kernel_libraries(self, dtype):
        return {"recurrent"} | ({"gemm_f32"} if dtype == torch.float32 else {"skinny_gemm"})

    def cache_need(self):
        return StateNeed((self.state_floats,), torch.float32)

    def bind(self, tensors, dtype, device):
        t = lambda logical: tensors[self.file_name(logical)]
        self.proj_weight = torch.cat((t("q_weight"), t("k_weight"), t("v_weight"), t("g_weight")), dim=0).contiguous()
        self.a1, self.a2 = t("a1").contiguous(), t("a2").contiguous()
        self.rank = int(self.a1.shape[0])
        self.a2_bias = t("a2_bias").to(torch.float32).contiguous()
        self.norm = t("norm").repeat(self.n_heads).contiguous()      # the one weight [vdim] under every head
        self.o_weight = t("o_weight")

    def step_weights(self):
        return [self.proj_weight, self.a1, self.a2, self.a2_bias, self.norm, self.o_weight]

    def forward(self, x, ctx, site, writes_cache):
        if not writes_cache:
            raise ValueError("gated_linear_attention: a recurrent state cannot be read from another schedule entry")
        n, h, d, v = x.shape[0], self.n_heads, self.dim, self.vdim
        f32 = dict(dtype=torch.float32, device=x.device)
        if runs_side_by_side(x):   # few rows: the decays' two products beside the projections' one
            main, side = fork(x)
            with torch.cuda.stream(side):
                pre = _low_rank(x, self.a1, self.a2, None)
            proj = ops.linear_rows(x, self.proj_weight)
            join(main, side, pre)
        else:
            proj = ops.linear_rows(x, self.proj_weight)                                  # [T, q | k | v | g]
            pre = _low_rank(x, self.a1, self.a2, None)                                   # float32 sums
        y = torch.empty((n, h * v), **f32)   # (the scan forms the decays sigmoid(pre + b)^(1 / tau) on its way in)
        ops.outer_state_scan_rows(proj[:, :h * d], proj[:, h * d:2 * h * d], proj[:, 2 * h * d:2 * h * d + h * v], pre, ctx.cu_q,
                                  ctx.slots, site.storage, 0, h, d, v, d ** -0.5, y, decay_from=("sigmoid_root", self.a2_bias, self.tau))
        out = torch.empty((n, h * v), dtype=x.dtype, device=x.device)
        ops.gated_group_norm(y, proj[:, 2 * h * d + h * v:], self.norm, self.eps, out, h, h, "silu", False)
        return ops.linear_rows(out, self.o_weight)


register_part("mixer", "matrix_memory", MatrixMemory)
register_part("mixer", "time_mix", TimeMix)
register_part("mixer", "gated_linear_attention", GatedLinearAttention)
register_part("mixer", "state_space", StateSpace)
