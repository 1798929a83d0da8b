"""anna_b200: the quantized paged KV-cache path of Anna (TurboQuant append, paged gather, GQA decode) for B200.

Everything computes through ``libanna_b200_kv.so`` (hand-written CUDA for sm_100a, C ABI in
``include/anna_b200_kv.h``); there is no CPU fallback.
"""
from .attention import grouped_query_attention
from .cache import KVCacheConfig, Qwen3DynamicCache, Qwen3PageAllocator
from .fused_ops import (
    gqa_decode_fused_is_available,
    gqa_decode_splitkv_fused_is_available,
    gqa_decode_splitkv_fused_out_is_available,
    gqa_decode_splitkv_turboquant_fused_out_is_available,
    maybe_load_gated_delta_library,
    paged_gqa_decode_fused_is_available,
    run_gqa_decode_fused,
    run_gqa_decode_splitkv_fused,
    run_gqa_decode_splitkv_fused_out,
    run_gqa_decode_splitkv_turboquant_fused_out,
    run_paged_gqa_decode_fused,
)
from .pools import Qwen3PagedLayerAllocator, TurboQuantLayerPool, resolve_value_group_size
from .prefix_block_cache import PrefixBlockPool
from .turboquant import VALID_KV_CACHE_QUANT_BITS, TurboQuantKVRow, TurboQuantTensorRow, turboquant_is_available

__all__ = [
    "KVCacheConfig", "Qwen3DynamicCache", "Qwen3PageAllocator", "Qwen3PagedLayerAllocator", "TurboQuantLayerPool",
    "PrefixBlockPool", "TurboQuantKVRow", "TurboQuantTensorRow", "VALID_KV_CACHE_QUANT_BITS", "resolve_value_group_size",
    "turboquant_is_available", "maybe_load_gated_delta_library", "gqa_decode_fused_is_available",
    "gqa_decode_splitkv_fused_is_available", "gqa_decode_splitkv_fused_out_is_available",
    "gqa_decode_splitkv_turboquant_fused_out_is_available", "paged_gqa_decode_fused_is_available",
    "run_gqa_decode_fused", "run_gqa_decode_splitkv_fused", "run_gqa_decode_splitkv_fused_out",
    "run_gqa_decode_splitkv_turboquant_fused_out", "run_paged_gqa_decode_fused", "grouped_query_attention",
]
