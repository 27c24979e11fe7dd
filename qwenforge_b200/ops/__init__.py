from .kernels import (TC_PLAIN, TC_SWIGLU, tc_gemm, tc_gemm_takes, tc_gemm_is_persistent, tc_gemm_qkv, tc_gemm_qkv_takes, rope_table, SampleScratch, EPI_PLAIN, EPI_QKV, EPI_RESIDUAL, EPI_SWIGLU, SKINNY_MAX_ROWS, residual_add, skinny_gemm, FusedProduct, skinny_chain, skinny_chain_takes, skinny_chain_repeated, wide_gemm, wide_gemm_takes, wide_gemm_takes_rows, residual_product_way, WIDE_MAX_ROWS, ERR_BARRIER_TIMEOUT,
                      skinny_gemm_takes, skinny_gemm_pays, decode_advance, decode_advance_embed, FAST_ATTENTION_HEAD_DIMS, GENERIC_DECODE_CHUNK, DecodeScratch, attention_decode, attention_decode_plan, attention_decode_warps, fold_project, fold_project_pays, fold_project_takes, attention_prefill, attention_prefill_tc, TC_ATTENTION_HEAD_DIMS, ERR_NO_PAGE, ERR_ROW_RANGE, ERR_TOKEN_RANGE, KernelError, KvSiteArgs, add_rms_norm,
                      attention_generic, describe_error_word, embed_gather, gather_rows, gather_rows_norm, gemm_f32, require_cuda,
                      rope_cache_write, sample, sm_count, swiglu, embed_positions, sandwich_norm, clamped_glu,
                      latent_norm_cache, head_linear, MoePlan, moe_plan, moe_gather, moe_combine, expert_linear, scaled_swiglu, tc_gemm_grouped, tc_gemm_grouped_takes, expert_gate_up, expert_gate_takes, moe_tile_rows, MOE_FUSED_ROUTER_MAX,
                      ERR_POSITION_RANGE, GENERIC_MAX_HEAD_DIM, bias_act, softcap_, stabilized_gates, decay_gates, outer_state_scan,
                      gated_group_norm, causal_conv_silu, OUTER_STATE_MAX_DIM, CONV_MAX_TAPS, ACTIVATIONS,
                      add_dyt_norm, add_dyt_norm_shift, residual_add_pair, stream_pair, head_gate, pool_cache_write, causal_conv,
                      add_rms_norm_scaled, residual_add_scaled, rms_norm_cols, mix_rows, bias_glu, shift_mix, channel_decay,
                      outer_state_scan_rows, rows_prepare)
from .linear import linear, linear_rows, gated_rows, own_tensor_core_products, use_own_tensor_core_products

__all__ = [
    "add_rms_norm_scaled", "residual_add_scaled", "rms_norm_cols", "mix_rows", "bias_glu", "shift_mix", "channel_decay",
    "outer_state_scan_rows", "rows_prepare",
    "add_dyt_norm", "add_dyt_norm_shift", "residual_add_pair", "stream_pair", "head_gate", "pool_cache_write", "causal_conv",
    "bias_act", "softcap_", "stabilized_gates", "decay_gates", "outer_state_scan", "gated_group_norm", "causal_conv_silu",
    "OUTER_STATE_MAX_DIM", "CONV_MAX_TAPS", "ACTIVATIONS",
    "embed_positions", "sandwich_norm", "clamped_glu", "latent_norm_cache", "head_linear", "MoePlan", "moe_plan", "moe_gather",
    "moe_combine", "expert_linear", "ERR_POSITION_RANGE", "GENERIC_MAX_HEAD_DIM", "scaled_swiglu", "moe_tile_rows",
    "MOE_FUSED_ROUTER_MAX", "linear_rows", "gated_rows", "tc_gemm_grouped", "tc_gemm_grouped_takes", "expert_gate_up", "expert_gate_takes",
    "ERR_NO_PAGE", "ERR_ROW_RANGE", "ERR_TOKEN_RANGE", "KernelError", "KvSiteArgs", "add_rms_norm",
    "attention_generic", "describe_error_word", "embed_gather", "gather_rows", "gather_rows_norm", "gemm_f32", "rope_cache_write",
    "sample", "swiglu", "linear", "own_tensor_core_products", "use_own_tensor_core_products", "require_cuda", "FAST_ATTENTION_HEAD_DIMS", "GENERIC_DECODE_CHUNK", "DecodeScratch",
    "attention_decode", "attention_decode_plan", "attention_decode_warps", "fold_project", "fold_project_pays", "fold_project_takes", "attention_prefill", "attention_prefill_tc", "TC_ATTENTION_HEAD_DIMS", "decode_advance", "decode_advance_embed", "EPI_PLAIN", "EPI_QKV", "EPI_RESIDUAL", "EPI_SWIGLU",
    "SKINNY_MAX_ROWS", "SampleScratch", "TC_PLAIN", "TC_SWIGLU", "tc_gemm", "tc_gemm_takes", "tc_gemm_is_persistent", "tc_gemm_qkv", "tc_gemm_qkv_takes", "rope_table", "residual_add", "skinny_gemm", "skinny_gemm_takes", "skinny_gemm_pays", "sm_count", "FusedProduct", "skinny_chain", "skinny_chain_takes", "skinny_chain_repeated", "ERR_BARRIER_TIMEOUT", "wide_gemm", "wide_gemm_takes", "wide_gemm_takes_rows", "residual_product_way", "WIDE_MAX_ROWS",
]
