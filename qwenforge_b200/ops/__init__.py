from .kernels import (TC_PLAIN, TC_SWIGLU, tc_gemm, tc_gemm_takes, tc_gemm_is_persistent, tc_gemm_qkv, tc_gemm_qkv_takes, rope_table, SampleScratch, EPI_PLAIN, EPI_QKV, EPI_RESIDUAL, EPI_SWIGLU, SKINNY_MAX_ROWS, residual_add, skinny_gemm, FusedProduct, skinny_chain, skinny_chain_takes, skinny_chain_repeated, wide_gemm, wide_gemm_takes, wide_gemm_takes_rows, residual_product_way, WIDE_MAX_ROWS, ERR_BARRIER_TIMEOUT,
                      skinny_gemm_takes, skinny_gemm_pays, decode_advance, decode_advance_embed, FAST_ATTENTION_HEAD_DIMS, GENERIC_DECODE_CHUNK, DecodeScratch, attention_decode, attention_decode_plan, attention_decode_warps, fold_project, fold_project_pays, fold_project_takes, attention_prefill, attention_prefill_tc, TC_ATTENTION_HEAD_DIMS, ERR_NO_PAGE, ERR_ROW_RANGE, ERR_TOKEN_RANGE, KernelError, KvSiteArgs, add_rms_norm,
                      attention_generic, describe_error_word, embed_gather, gather_rows, gather_rows_norm, gemm_f32, require_cuda,
                      rope_cache_write, sample, sm_count, swiglu)
from .linear import linear, own_tensor_core_products, use_own_tensor_core_products

__all__ = [
    "ERR_NO_PAGE", "ERR_ROW_RANGE", "ERR_TOKEN_RANGE", "KernelError", "KvSiteArgs", "add_rms_norm",
    "attention_generic", "describe_error_word", "embed_gather", "gather_rows", "gather_rows_norm", "gemm_f32", "rope_cache_write",
    "sample", "swiglu", "linear", "own_tensor_core_products", "use_own_tensor_core_products", "require_cuda", "FAST_ATTENTION_HEAD_DIMS", "GENERIC_DECODE_CHUNK", "DecodeScratch",
    "attention_decode", "attention_decode_plan", "attention_decode_warps", "fold_project", "fold_project_pays", "fold_project_takes", "attention_prefill", "attention_prefill_tc", "TC_ATTENTION_HEAD_DIMS", "decode_advance", "decode_advance_embed", "EPI_PLAIN", "EPI_QKV", "EPI_RESIDUAL", "EPI_SWIGLU",
    "SKINNY_MAX_ROWS", "SampleScratch", "TC_PLAIN", "TC_SWIGLU", "tc_gemm", "tc_gemm_takes", "tc_gemm_is_persistent", "tc_gemm_qkv", "tc_gemm_qkv_takes", "rope_table", "residual_add", "skinny_gemm", "skinny_gemm_takes", "skinny_gemm_pays", "sm_count", "FusedProduct", "skinny_chain", "skinny_chain_takes", "skinny_chain_repeated", "ERR_BARRIER_TIMEOUT", "wide_gemm", "wide_gemm_takes", "wide_gemm_takes_rows", "residual_product_way", "WIDE_MAX_ROWS",
]
