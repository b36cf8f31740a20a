"""Operators of this package (reference: src/flaggems_vllm/ops/__init__.py:61-63,191)."""
from .act_quant import act_quant_triton
from .cp_gather_indexer_k_quant_cache import cp_gather_indexer_k_quant_cache
from .deepseek_v4_attention_combine_topk_swa_indices import combine_topk_swa_indices
from .deepseek_v4_attention_compute_global_topk_indices_and_lens import compute_global_topk_indices_and_lens
from .deepseek_v4_attention_dequantize_and_gather_k_cache import dequantize_and_gather_k_cache
from .deepseek_v4_attention_fused_q_kv_rmsnorm import fused_q_kv_rmsnorm
from .fused_deepseek_v4_qnorm_rope_kv_rope_quant_insert import (
    fused_deepseek_v4_qnorm_rope_kv_rope_quant_insert,
    fused_deepseek_v4_qnorm_rope_kv_rope_quant_insert_checked,
    fused_deepseek_v4_qnorm_rope_kv_rope_quant_insert_padded,
)
from .fused_indexer_q_rope_quant import fused_indexer_q_rope_quant
from .fused_inv_rope_fp8_quant import fused_inv_rope_fp8_quant
from .gather_dequant_k_cache import gather_dequant_k_cache_slots
from .host_staged import HostStagedPrologue
from .indexer_k_quant_and_cache import indexer_k_quant_and_cache
from .per_token_group_quant_fp8 import per_token_group_quant_fp8
from .persistent_topk import persistent_topk
from .top_k_per_row_decode import top_k_per_row_decode
from .top_k_per_row_prefill import top_k_per_row_prefill

__all__ = [
    "fused_indexer_q_rope_quant",
    "indexer_k_quant_and_cache",
    "cp_gather_indexer_k_quant_cache",
    "combine_topk_swa_indices",
    "compute_global_topk_indices_and_lens",
    "per_token_group_quant_fp8",
    "act_quant_triton",
    "persistent_topk",
    "top_k_per_row_decode",
    "top_k_per_row_prefill",
    "fused_inv_rope_fp8_quant",
    "fused_q_kv_rmsnorm",
    "dequantize_and_gather_k_cache",
    "fused_deepseek_v4_qnorm_rope_kv_rope_quant_insert",
    "fused_deepseek_v4_qnorm_rope_kv_rope_quant_insert_checked",
    "fused_deepseek_v4_qnorm_rope_kv_rope_quant_insert_padded",
    "gather_dequant_k_cache_slots",
    "HostStagedPrologue",
]
