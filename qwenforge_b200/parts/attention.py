"""Grouped-query softmax attention over the cache (student_engine.py:556-599, :795-832).

  qkv = x Wqkv^T + bqkv            one product on the row-concatenated q, k, v weights (:505-520)
  q, k rotated by position         the position part; fused into the cache-write kernel when it is rotary
  k, v appended to the cache       at the token's own position of its own sequence
  ctx = softmax(q k^T * scale) v   query head i reads kv head i // (NH / KVH); key j visible iff
                                   max(0, p - window + 1) <= j <= p for a query at position p
  out = ctx Wo^T (+ bo)

Nothing here is specific to one model: head counts, head size, biases, scale, window and the
position part all come from the spec. A step's queries attend to the cache only, which already
holds the step's own keys: whole prompts, continuations and single tokens are the same code.

Options that other designs switch on, each a parameter of the spec (all off for the plain form above):
  value_dim      values of another size than keys. The smaller of the two is padded with zeros up to the larger in the
                 projection weights, once at load time, so that the cache and the kernels see one head size; zeros add
                 nothing to a score and come out as zeros.
  unit_norm_eps  after the rotation, q and k are divided by their root mean square per head (no weight)
  softcap        score <- softcap * tanh(score / softcap), after the scale
  chunk          key j is visible to query i only inside i's block of `chunk` positions (counted from position 0)
  sink           "unit": one more term exp(0) in the softmax's denominator, with no value
  own_kv         false: no key and value projections; the layer reads the cache of the schedule entry it is pointed at
  conv_taps      a short causal convolution over time on every channel of q, k and v, right after the projection
                 (y_t = sum_j c[:, j] u_(t - taps + 1 + j), no bias, zeros before a sequence's start); the last taps - 1
                 projected rows of a sequence are part of its state
  qk_norm_eps    q and k are RMS-normed per head BEFORE the rotation, with a weight each (`q_norm`, `k_norm`: [head_dim],
                 shared by the heads)
  sink           "learned": exp(sink_h) joins the softmax's denominator, a number per head from the weight files
  pool           with a window: one pooled key and value for every block of `pool` positions that lies wholly before the
                 query's window (block b is seen from position b * pool + pool - 1 + window on), the means of the block's
                 keys and values as the cache holds them, in the same softmax. They live in a second paged cache of one row
                 per block; the positions themselves stay until their block is complete
  head_gate      every head's output is multiplied by sigmoid(G h)_head, one more projection [heads, hidden] of the same input
  row_norm_eps   q and k are RMS-normed over their WHOLE rows (all heads at once: the mean over heads * head_dim numbers),
                 after the biases and before the rotation, with a weight per column (`q_row_norm` [heads * head_dim],
                 `k_row_norm` [kv_heads * head_dim])
  value_mix      {"role": "source" | "mix", "key": name}: the layers that share a key form a chain through one step. The
                 source keeps its values (after the bias) for the others; a "mix" layer replaces its own by
                 (1 - l) v + l v_source of the same token, l a learned number (`value_mix`), and caches the mixed values
The position part may pair components 2j and 2j + 1 (`rotary_interleaved`) instead of j and j + R/2.
"""
from __future__ import annotations

import torch

from .. import ops
from ..cache import PAGE_TOKENS, BundleNeed, KvNeed, StateNeed
from .base import Mixer, TensorSpec
from .registry import build_part, register_part


# Fewest new tokens of a step, by head size, from which the tcgen05 prefill attention runs instead of the mma.sync one.
# Measured on one prompt (`python -m qwenforge_b200.measure attention`): head size 64, 14 heads: 17 against 21
# microseconds at 1,024 tokens, 27 against 42 at 2,048, 72 against 116 at 4,096, 199 against 415 at 8,192 (at 512 tokens
# 15 against 13); head size 128, 16 heads: 16 against 17 at 512 tokens, 24 against 36 at 1,024, 52 against 72 at 2,048,
# 140 against 245 at 4,096. Below, its tiles of 128 rows are too few to fill the SMs.
TC_PREFILL_MIN_TOKENS = {64: 1024, 128: 512}


class GqaAttention(Mixer):
    """params: hidden_size, num_heads, num_kv_heads, head_dim, qkv_bias, out_bias, scale, window, position (PartSpec | None),
    and optionally value_dim, unit_norm_eps, softcap, chunk, sink, own_kv (see the top of the file).
    tensors: q_weight, k_weight, v_weight, o_weight (+ q_bias, k_bias, v_bias, o_bias when enabled)."""

    def __init__(self, spec):
        super().__init__(spec)
        p = self.params
        self.hidden = int(p["hidden_size"])
        self.n_heads = int(p["num_heads"])
        self.n_kv = int(p["num_kv_heads"])
        self.key_dim = int(p["head_dim"])
        self.value_dim = int(p.get("value_dim") or self.key_dim)
        self.head_dim = max(self.key_dim, self.value_dim)   # what the cache and the kernels see
        self.unit_norm_eps = None if p.get("unit_norm_eps") is None else float(p["unit_norm_eps"])
        self.softcap = float(p.get("softcap") or 0.0)
        self.chunk = int(p.get("chunk") or 0)
        self.sink = str(p.get("sink") or "none")
        self.own_kv = bool(p.get("own_kv", True))
        self.conv_taps = int(p.get("conv_taps") or 0)
        self.qk_norm_eps = None if p.get("qk_norm_eps") is None else float(p["qk_norm_eps"])
        self.pool = int(p.get("pool") or 0)
        self.gated = bool(p.get("head_gate", False))
        self.row_norm_eps = None if p.get("row_norm_eps") is None else float(p["row_norm_eps"])
        self.value_mix = dict(p["value_mix"]) if p.get("value_mix") else None
        if self.value_mix is not None and (self.value_mix.get("role") not in ("source", "mix") or not p.get("own_kv", True)):
            raise ValueError("gqa_attention: value_mix has the role 'source' or 'mix' and goes with values of the layer's own")
        if self.row_norm_eps is not None and (p.get("qk_norm_eps") is not None or int(p.get("conv_taps") or 0) > 0 or not p.get("own_kv", True)):
            raise ValueError("gqa_attention: a norm over whole rows goes with keys of the layer's own, without a norm per head "
                             "before the rotation and without a short convolution")
        if self.sink not in ("none", "unit", "learned"):
            raise ValueError(f"gqa_attention: sink {self.sink!r} is not known ('none', 'unit' or 'learned')")
        if self.unit_norm_eps is not None and self.qk_norm_eps is not None:
            raise ValueError("gqa_attention: a norm of q and k comes either before the rotation (qk_norm_eps) or after it (unit_norm_eps)")
        if self.pool > 0 and (int(p.get("window") or 0) <= 0 or self.chunk > 0 or not self.own_kv):
            raise ValueError("gqa_attention: pooled blocks go with a window, without a block mask, in a layer with keys of its own")
        if self.conv_taps > ops.CONV_MAX_TAPS or (self.conv_taps > 0 and (not self.own_kv or p.get("qkv_bias"))):
            raise ValueError(f"gqa_attention: a short convolution has up to {ops.CONV_MAX_TAPS} taps and goes with q, k and v "
                             "of the layer's own, without biases")
        self.interleaved = bool(p.get("position") is not None and p["position"].kind == "rotary_interleaved")
        # the form that every tensor-core kernel and fused product of this part takes
        self.plain = (self.value_dim == self.key_dim and self.unit_norm_eps is None and self.softcap == 0.0 and self.chunk == 0
                      and self.sink == "none" and self.own_kv and self.conv_taps == 0 and self.qk_norm_eps is None
                      and self.pool == 0 and not self.gated and not self.interleaved and self.row_norm_eps is None
                      and self.value_mix is None)
        self.qkv_bias = bool(p.get("qkv_bias", False))
        self.out_bias = bool(p.get("out_bias", False))
        self.scale = float(p.get("scale") or self.key_dim ** -0.5)
        self.window = int(p.get("window") or 0)
        if self.n_heads % self.n_kv:
            raise ValueError(f"gqa_attention: {self.n_heads} heads are not divisible by {self.n_kv} kv heads")
        if self.head_dim > 256:
            raise ValueError(f"gqa_attention: head_dim {self.head_dim} > 256 is not supported by the attention kernels")
        self.position = build_part("position", p["position"]) if p.get("position") is not None else None
        self.q_width = self.n_heads * self.head_dim
        self.kv_width = self.n_kv * self.head_dim
        self.qkv_width = self.q_width + (2 * self.kv_width if self.own_kv else 0)   # the gates' columns follow
        self.qkv_weight = self.qkv_bias_t = self.o_weight = self.o_bias_t = self.sinks = None
        self.conv_weight = self.q_norm = self.k_norm = self.q_row_norm = self.k_row_norm = None
        self.mix_weight = 0.0

    def sub_parts(self):
        return [self.position] if self.position is not None else []

    def tensor_specs(self):
        kd, vd = self.key_dim, self.value_dim
        specs = [TensorSpec(self.file_name("q_weight"), (self.n_heads * kd, self.hidden))]
        if self.own_kv:
            specs += [TensorSpec(self.file_name("k_weight"), (self.n_kv * kd, self.hidden)),
                      TensorSpec(self.file_name("v_weight"), (self.n_kv * vd, self.hidden))]
        specs.append(TensorSpec(self.file_name("o_weight"), (self.hidden, self.n_heads * vd)))
        if self.qkv_bias:
            specs.append(TensorSpec(self.file_name("q_bias"), (self.n_heads * kd,), init="bias"))
            if self.own_kv:
                specs += [TensorSpec(self.file_name("k_bias"), (self.n_kv * kd,), init="bias"),
                          TensorSpec(self.file_name("v_bias"), (self.n_kv * vd,), init="bias")]
        if self.out_bias:
            specs.append(TensorSpec(self.file_name("o_bias"), (self.hidden,), init="bias"))
        if self.conv_taps > 0:
            specs += [TensorSpec(self.file_name("q_conv"), (self.n_heads * kd, self.conv_taps), init="conv", keep="float32"),
                      TensorSpec(self.file_name("k_conv"), (self.n_kv * kd, self.conv_taps), init="conv", keep="float32"),
                      TensorSpec(self.file_name("v_conv"), (self.n_kv * vd, self.conv_taps), init="conv", keep="float32")]
        if self.qk_norm_eps is not None:
            specs += [TensorSpec(self.file_name("q_norm"), (kd,), init="norm"), TensorSpec(self.file_name("k_norm"), (kd,), init="norm")]
        if self.sink == "learned":
            specs.append(TensorSpec(self.file_name("sink"), (self.n_heads,), init="logit", keep="float32"))
        if self.gated:
            specs.append(TensorSpec(self.file_name("g_weight"), (self.n_heads, self.hidden)))
        if self.row_norm_eps is not None:
            specs += [TensorSpec(self.file_name("q_row_norm"), (self.n_heads * kd,), init="norm"),
                      TensorSpec(self.file_name("k_row_norm"), (self.n_kv * kd,), init="norm")]
        if self.value_mix is not None and self.value_mix["role"] == "mix":
            specs.append(TensorSpec(self.file_name("value_mix"), (), init="fraction", keep="float32"))
        return specs

    def kernel_libraries(self, dtype):
        libs = {"rope_cache", "attention_generic"} | ({"recurrent"} if self.conv_taps > 0 else set()) \
            | ({"activation"} if self.gated else set()) | ({"norm"} if self.row_norm_eps is not None or self.value_mix else set())
        if dtype == torch.float32:
            libs.add("gemm_f32")
        elif not self.plain and self.head_dim in ops.FAST_ATTENTION_HEAD_DIMS:
            libs |= {"attention_decode", "attention_prefill", "skinny_gemm"}
        elif self.head_dim in ops.FAST_ATTENTION_HEAD_DIMS:
            libs |= {"attention_decode", "attention_prefill", "skinny_gemm", "wide_gemm", "fold_project"}
            if self.head_dim in ops.TC_ATTENTION_HEAD_DIMS:
                libs.add("attention_prefill_tc")
        return libs

    def cache_need(self):
        kv = KvNeed(self.n_kv, self.head_dim, self.window, chunk=self.chunk, pool=self.pool)
        if self.pool <= 0 and self.conv_taps <= 0:
            return kv
        items = [("kv", kv)]
        if self.pool > 0:
            items.append(("blocks", KvNeed(self.n_kv, self.head_dim, every=self.pool)))
        if self.conv_taps > 0:   # (a convolution of one tap keeps nothing; its row is never read or written)
            items.append(("conv", StateNeed((max(self.conv_taps - 1, 1) * self.qkv_width,), torch.float32)))
        return BundleNeed(tuple(items))

    def _padded(self, rows: torch.Tensor, heads: int, size: int) -> torch.Tensor:
        """Rows [heads * size, ...] of a projection (or its bias) with every head filled up with zero rows to head_dim."""
        if size == self.head_dim:
            return rows
        wide = rows.new_zeros((heads, self.head_dim) + tuple(rows.shape[1:]))
        wide[:, :size] = rows.view((heads, size) + tuple(rows.shape[1:]))
        return wide.view((heads * self.head_dim,) + tuple(rows.shape[1:]))

    def bind(self, tensors, dtype, device):
        t = lambda logical: tensors[self.file_name(logical)]
        kd, vd = self.key_dim, self.value_dim
        pieces = [self._padded(t("q_weight"), self.n_heads, kd)]
        if self.own_kv:
            pieces += [self._padded(t("k_weight"), self.n_kv, kd), self._padded(t("v_weight"), self.n_kv, vd)]
        if self.gated:   # the gates' logits are further columns of the one product
            pieces.append(t("g_weight"))
            rows = sum(p.shape[0] for p in pieces)
            if rows % 8:   # zero rows up to a row pitch of whole 16 bytes: the library's products choose their kernels by it
                pieces.append(pieces[0].new_zeros((8 - rows % 8, pieces[0].shape[1])))
        self.qkv_weight = torch.cat(pieces, dim=0).contiguous()
        if self.conv_taps > 0:   # zero taps under the padding: what is zero stays zero
            self.conv_weight = torch.cat((self._padded(t("q_conv"), self.n_heads, kd), self._padded(t("k_conv"), self.n_kv, kd),
                                          self._padded(t("v_conv"), self.n_kv, vd)), dim=0).to(torch.float32).contiguous()
        if self.qk_norm_eps is not None:
            self.q_norm, self.k_norm = t("q_norm").contiguous(), t("k_norm").contiguous()
        if self.row_norm_eps is not None:   # (zero weights under the padding, where the rows hold zeros anyway)
            self.q_row_norm = self._padded(t("q_row_norm"), self.n_heads, kd).contiguous()
            self.k_row_norm = self._padded(t("k_row_norm"), self.n_kv, kd).contiguous()
        if self.value_mix is not None and self.value_mix["role"] == "mix":
            self.mix_weight = float(t("value_mix").float().item())   # a scalar, read once when the weights are bound
        if self.qkv_bias:
            pieces = [self._padded(t("q_bias"), self.n_heads, kd)]
            if self.own_kv:
                pieces += [self._padded(t("k_bias"), self.n_kv, kd), self._padded(t("v_bias"), self.n_kv, vd)]
            self.qkv_bias_t = torch.cat(pieces, dim=0).contiguous()
        o = t("o_weight")
        if vd != self.head_dim:   # columns of zeros under the attended heads' padding
            o = self._padded(o.t().contiguous(), self.n_heads, vd).t().contiguous()
        self.o_weight = o
        if self.out_bias:
            self.o_bias_t = t("o_bias")
        if self.sink == "unit":
            self.sinks = torch.zeros(self.n_heads, dtype=torch.float32, device=device)
        elif self.sink == "learned":
            self.sinks = t("sink").to(torch.float32).contiguous()

    def step_weights(self):
        return [t for t in (self.qkv_weight, self.qkv_bias_t, self.o_weight, self.o_bias_t, self.conv_weight, self.q_norm,
                            self.k_norm, self.q_row_norm, self.k_row_norm) if t is not None]

    def forward(self, x, ctx, site, writes_cache):
        n = x.shape[0]
        if not self.plain:
            return self._forward_with_options(x, ctx, site, writes_cache)
        fast = (ctx.attention == "auto" and x.dtype == torch.bfloat16
                and self.head_dim in ops.FAST_ATTENTION_HEAD_DIMS)
        plan = self.decode_plan(ctx) if fast and ctx.is_decode else None
        rotary = self.position.fused_rotary() if self.position is not None else None
        # (The product with bias, rotation and cache write in its epilogue, `ops.tc_gemm_qkv`, was measured inside the
        # prompt graph of 2,048 tokens at Qwen2.5-0.5B sizes: 2.88 ms for the step against 2.76 with the library product
        # and the rotation kernel; it is not used here.)
        late_bias = self.position is None or rotary is not None  # the kernel that rotates and stores adds the bias
        qkv = ops.linear(x, self.qkv_weight, None if late_bias else self.qkv_bias_t)
        if self.position is not None and rotary is None:
            q_view = qkv[:, :self.q_width].view(n, self.n_heads, self.head_dim)
            k_view = qkv[:, self.q_width:self.q_width + self.kv_width].view(n, self.n_kv, self.head_dim)
            self.position.apply(q_view, k_view, ctx)
        inv_freq, rot_dim = rotary if rotary is not None else (None, 0)
        q = torch.empty((n, self.q_width), dtype=x.dtype, device=x.device)
        args = ops.KvSiteArgs(site.storage, site.table, self.n_kv, self.head_dim)
        ops.rope_cache_write(qkv, ctx.tok_seq, ctx.tok_pos, ctx.slots, inv_freq, rot_dim, self.n_heads, q, args,
                             writes_cache, ctx.err, bias=self.qkv_bias_t if late_bias else None)
        attended = torch.empty_like(q)
        if fast and ctx.is_decode:
            ops.attention_decode(q, attended, ctx.cu_q, ctx.tok_pos, ctx.slots, args, self.n_heads, ctx.n_seqs,
                                 self.scale, self.window, self.decode_splits(ctx), ctx.decode_scratch, ctx.err, plan)
        elif fast:
            # the tcgen05 kernel works on blocks of 128 query rows, a long chain of pages per block: it pays for steps
            # with many rows
            least = TC_PREFILL_MIN_TOKENS.get(self.head_dim)
            prefill = (ops.attention_prefill_tc if least is not None and n >= least and ctx.max_q_len >= 128
                       else ops.attention_prefill)
            prefill(q, attended, ctx.cu_q, ctx.tok_pos, ctx.slots, args, self.n_heads, ctx.n_seqs,
                    ctx.max_q_len, self.scale, self.window, ctx.err, max_kv_len=ctx.max_kv_len)
        else:
            ops.attention_generic(q, attended, ctx.cu_q, ctx.tok_pos, ctx.slots, args, self.n_heads, ctx.n_seqs,
                                  ctx.max_q_len, self.scale, self.window, ctx.err, scratch=ctx.decode_scratch,
                                  max_kv_len=ctx.max_kv_len)
        return ops.linear(attended, self.o_weight, self.o_bias_t)

    def _forward_with_options(self, x, ctx, site, writes_cache):
        """The step with any of the options on: one product for what the layer projects, the short convolution, one kernel
        for bias, norms, rotation and the cache write, the pooled rows of the blocks that the step completed, then attention
        over the cache with the mask, the cap, the pooled rows and the sink, the heads' gates, the output projection."""
        n = x.shape[0]
        if self.position is not None and self.position.fused_rotary() is None:
            raise ValueError("gqa_attention: the options need a position part with a fused form (or none)")
        if not self.own_kv and writes_cache:
            raise ValueError("gqa_attention: a layer without keys and values of its own must be pointed at another entry's cache")
        bundled = self.pool > 0 or self.conv_taps > 0
        if bundled and not writes_cache:
            raise ValueError("gqa_attention: a layer with a convolution's state or pooled rows cannot read another entry's cache")
        kv_site = site["kv"] if bundled else site
        inv_freq, rot_dim = self.position.fused_rotary() if self.position is not None else (None, 0)
        late_bias = self.qkv_bias_t
        if self.row_norm_eps is not None or self.value_mix is not None:
            # what follows reads q, k and v with their biases: the bias joins the product, not the rotation kernel
            # (biases, both norms and the values' mixing are one kernel behind the product)
            qkv = ops.linear_rows(x, self.qkv_weight)
            late_bias = None
            self._prepare_rows(qkv, ctx)
        else:
            qkv = ops.linear_rows(x, self.qkv_weight)           # [T, q | k | v (| gates)]
        gates = qkv[:, self.qkv_width:self.qkv_width + self.n_heads] if self.gated else None
        if self.conv_taps > 0:
            mixed = torch.empty((n, self.qkv_width), dtype=x.dtype, device=x.device)
            ops.causal_conv(qkv[:, :self.qkv_width], self.conv_weight, None, ctx.cu_q, ctx.tok_seq, ctx.slots, site["conv"].storage,
                            0, mixed, single=ctx.is_decode and n == ctx.n_seqs)
            qkv = mixed
        q = torch.empty((n, self.q_width), dtype=x.dtype, device=x.device)
        args = ops.KvSiteArgs(kv_site.storage, kv_site.table, self.n_kv, self.head_dim)
        norm_first = self.qk_norm_eps is not None
        ops.rope_cache_write(qkv, ctx.tok_seq, ctx.tok_pos, ctx.slots, inv_freq, rot_dim, self.n_heads, q, args, writes_cache,
                             ctx.err, bias=late_bias, unit_norm_eps=self.qk_norm_eps if norm_first else self.unit_norm_eps,
                             norm_dim=self.key_dim, has_kv=self.own_kv, interleaved=self.interleaved, norm_first=norm_first,
                             q_norm=self.q_norm, k_norm=self.k_norm)
        blocks = None
        if self.pool > 0:
            blocks = ops.KvSiteArgs(site["blocks"].storage, site["blocks"].table, self.n_kv, self.head_dim)
            ops.pool_cache_write(ctx.cu_q, ctx.tok_pos, ctx.slots, args, blocks, self.pool, ctx.max_q_len, ctx.err)
        attended = torch.empty_like(q)
        fast = ctx.attention == "auto" and x.dtype == torch.bfloat16 and self.head_dim in ops.FAST_ATTENTION_HEAD_DIMS
        # (pooled rows: single tokens run on the kernel of portions too. What a token reads there is bounded by its window
        # and a row per block before it, a few pages that need no cut into runs; the split-K kernel does not take the rows.)
        if fast and ctx.is_decode and n == ctx.n_seqs and self.pool == 0:
            n_splits = self.decode_splits(ctx)
            ops.attention_decode(q, attended, ctx.cu_q, ctx.tok_pos, ctx.slots, args, self.n_heads, ctx.n_seqs, self.scale,
                                 self.window, n_splits, ctx.decode_scratch, ctx.err, self.decode_plan(ctx), sinks=self.sinks,
                                 chunk=self.chunk, softcap=self.softcap)
        elif fast:
            ops.attention_prefill(q, attended, ctx.cu_q, ctx.tok_pos, ctx.slots, args, self.n_heads, ctx.n_seqs, ctx.max_q_len,
                                  self.scale, self.window, ctx.err, max_kv_len=ctx.max_kv_len, sinks=self.sinks,
                                  chunk=self.chunk, softcap=self.softcap, blocks=blocks, pool=self.pool)
        else:
            ops.attention_generic(q, attended, ctx.cu_q, ctx.tok_pos, ctx.slots, args, self.n_heads, ctx.n_seqs, ctx.max_q_len,
                                  self.scale, self.window, ctx.err, scratch=ctx.decode_scratch, max_kv_len=ctx.max_kv_len,
                                  sinks=self.sinks, chunk=self.chunk, softcap=self.softcap, blocks=blocks, pool=self.pool)
        if self.gated:
            ops.head_gate(attended, gates, self.n_heads)
        return ops.linear(attended, self.o_weight, self.o_bias_t) if self.o_bias_t is not None else ops.linear_rows(attended, self.o_weight)

    def _prepare_rows(self, qkv, ctx) -> None:
        """Biases, the norms of q and k over their whole rows and the chain of layers that share values, in one launch on the
        product's output: the chain's source leaves its values (a view of this output, kept alive by the step's memo) for
        the layers after it; a mixing layer draws its own towards them in place."""
        q_w, kv_w, b = self.q_width, self.kv_width, self.qkv_bias_t
        piece = lambda lo, hi: None if b is None else b[lo:hi]
        normed = self.row_norm_eps is not None
        runs = [(0, q_w, self.n_heads * self.key_dim if normed else 0, piece(0, q_w), self.q_row_norm),
                (q_w, kv_w, self.n_kv * self.key_dim if normed else 0, piece(q_w, q_w + kv_w), self.k_row_norm),
                (q_w + kv_w, kv_w, 0, piece(q_w + kv_w, q_w + 2 * kv_w), None)]
        mix = None
        if self.value_mix is not None:
            key = ("gqa_attention.value_mix", self.value_mix["key"])
            memo = ctx.step_memo if ctx.step_memo is not None else {}
            if self.value_mix["role"] == "source":
                memo[key] = (qkv[:, q_w + kv_w:q_w + 2 * kv_w], self.n_kv, self.value_dim, self.head_dim)
            else:
                if key not in memo:
                    raise RuntimeError("gqa_attention: a layer mixes in the values of a layer that has not run in this step")
                source, heads, size, source_head = memo[key]
                if (heads, size) != (self.n_kv, self.value_dim):
                    raise ValueError("gqa_attention: layers that mix their values have as many key/value heads of the same value size")
                mix = (2, source, self.value_dim, self.head_dim, source_head, self.mix_weight)
        ops.rows_prepare(qkv, runs, self.row_norm_eps if normed else 0.0, mix)

    # ---- the form for decode steps of up to 64 sequences that works on the residual stream in place: the norm, bias,
    # rotation and cache write ride on the QKV product and the addition on the output projection wherever a kernel of
    # this library takes the sizes and is the faster way by measurement; each product chooses for itself.
    def _ways(self, ctx):
        rows = ctx.n_tokens
        rotary = self.position.fused_rotary() if self.position is not None else None
        qkv = "unfused"
        if rows <= ops.SKINNY_MAX_ROWS and ops.skinny_gemm_takes(rows, self.qkv_weight, ops.EPI_QKV, True, n_heads=self.n_heads,
                                                                 kv_heads=self.n_kv, head_dim=self.head_dim,
                                                                 rot_dim=rotary[1] if rotary else 0):
            qkv = "skinny"
        return qkv, ops.residual_product_way(rows, self.o_weight)

    def fused_takes(self, ctx) -> bool:
        if not (self.plain and ctx.attention == "auto" and ctx.is_decode and ctx.dtype == torch.bfloat16
                and ctx.n_tokens <= ops.WIDE_MAX_ROWS and self.head_dim in ops.FAST_ATTENTION_HEAD_DIMS and not self.out_bias):
            return False
        rotary = self.position.fused_rotary() if self.position is not None else None
        if self.position is not None and (rotary is None or rotary[1] != self.head_dim):
            return False
        return self._ways(ctx) != ("unfused", "unfused")

    def fused_forward(self, hidden, rms, ctx, site, writes_cache, delta=None):
        n = hidden.shape[0]
        qkv_way, o_way = self._ways(ctx)
        plan = self.decode_plan(ctx)
        inv_freq, rot_dim = self.position.fused_rotary() if self.position is not None else (None, 0)
        args = ops.KvSiteArgs(site.storage, site.table, self.n_kv, self.head_dim)
        q = torch.empty((n, self.q_width), dtype=torch.bfloat16, device=hidden.device)
        if qkv_way == "skinny":
            if delta is not None:
                ops.residual_add(hidden, delta)
            ops.skinny_gemm(ops.EPI_QKV, self.qkv_weight, hidden=hidden, norm_weight=rms[0], eps=rms[1],
                            bias=self.qkv_bias_t,
                            qkv=dict(n_heads=self.n_heads, site=args, inv_freq=inv_freq, rot_dim=rot_dim, tok_pos=ctx.tok_pos,
                                     tok_seq=ctx.tok_seq, slots=ctx.slots, q_out=q, write_cache=writes_cache, err=ctx.err))
        else:
            x = torch.empty(hidden.shape, dtype=torch.bfloat16, device=hidden.device)
            ops.add_rms_norm(hidden, delta, rms[0], rms[1], x)   # the norm kernel adds the pending delta on its way
            ops.rope_cache_write(ops.linear(x, self.qkv_weight), ctx.tok_seq, ctx.tok_pos, ctx.slots, inv_freq, rot_dim,
                                 self.n_heads, q, args, writes_cache, ctx.err, bias=self.qkv_bias_t)
        n_splits = self.decode_splits(ctx)
        if (o_way == "skinny" and n == ctx.n_seqs and ops.fold_project_pays(n, self.o_weight)
                and ops.fold_project_takes(n, self.o_weight, hidden, self.n_heads, self.head_dim)):
            # the attention kernel stops at its runs' partial results; the projection folds them on its way in
            ops.attention_decode(q, None, ctx.cu_q, ctx.tok_pos, ctx.slots, args, self.n_heads, ctx.n_seqs, self.scale,
                                 self.window, n_splits, ctx.decode_scratch, ctx.err, plan, fold_later=True)
            ops.fold_project(plan, ctx.decode_scratch, self.o_weight, hidden, self.n_heads, self.head_dim, n_splits)
            return
        attended = torch.empty_like(q)
        ops.attention_decode(q, attended, ctx.cu_q, ctx.tok_pos, ctx.slots, args, self.n_heads, ctx.n_seqs,
                             self.scale, self.window, n_splits, ctx.decode_scratch, ctx.err, plan)
        if o_way == "skinny":
            ops.skinny_gemm(ops.EPI_RESIDUAL, self.o_weight, x=attended, residual=hidden)
        elif o_way == "wide":
            ops.wide_gemm(ops.EPI_RESIDUAL, self.o_weight, x=attended, residual=hidden, err=ctx.err)
        else:
            ops.residual_add(hidden, ops.linear(attended, self.o_weight))

    def decode_plan(self, ctx) -> torch.Tensor:
        """Which block of the decode attention takes which run of which sequence: made once per step, by the first
        layer of this shape that runs, and shared through the step's memo by the others."""
        n_splits = self.decode_splits(ctx)
        key = ("gqa_attention.decode_plan", self.n_kv, self.n_heads, self.head_dim, self.window, n_splits, self.chunk)
        memo = ctx.step_memo if ctx.step_memo is not None else {}
        plan = memo.get(key)
        if plan is None:
            plan = memo[key] = ops.attention_decode_plan(ctx.cu_q, ctx.tok_pos, ctx.slots, self.n_kv, self.head_dim,
                                                         self.n_heads, ctx.n_seqs, self.window, n_splits, ctx.decode_scratch,
                                                         self.chunk)
        return plan

    def decode_splits(self, ctx) -> int:
        """The most blocks that may share one (sequence, kv head): a block's warps take one page each
        (`ops.attention_decode_warps`), so at most one split per that many pages of the longest sequence that the step allows.
        How many of them a sequence gets is the kernel's decision, from the lengths on the device; this number sizes
        its grid and scratch and depends on the batch's shape only (fixed inside a captured graph)."""
        span = ctx.max_kv_len if self.window <= 0 else min(ctx.max_kv_len, self.window + PAGE_TOKENS)
        if self.chunk > 0:
            span = min(span, self.chunk + PAGE_TOKENS)
        pages = max(1, -(-span // PAGE_TOKENS))
        warps = ops.attention_decode_warps(self.head_dim)
        return max(1, min(-(-pages // warps), 64))


register_part("mixer", "gqa_attention", GqaAttention)
