"""Gather of the sparse-indexer keys and their scales from the paged cache into token order.

Drop-in for the reference operator of the same module path and name
(src/flaggems_vllm/ops/cp_gather_indexer_k_quant_cache.py:129-190): same arguments and in-place effect on
`k_fp8` and `k_fp8_scale`; rows beyond `cu_seqlen[-1]` are left untouched.  The cache is the one
`indexer_k_quant_and_cache` writes ([num_blocks, block_size, head_dim + 4*head_dim/quant_block_size] uint8:
per block all value bytes first, then all fp32 scales).
"""
from __future__ import annotations

import torch

from .. import _native


def cp_gather_indexer_k_quant_cache(k_cache: torch.Tensor, k_fp8: torch.Tensor, k_fp8_scale: torch.Tensor,
                                    block_table: torch.Tensor, cu_seqlen: torch.Tensor) -> None:
    num_tokens = k_fp8.size(0)
    block_size = k_cache.size(1)
    head_dim = k_fp8.shape[-1]
    num_blocks = k_cache.shape[0]
    # the reference takes the scales as uint8 [T, 4*groups]; a float32 [T, groups] tensor is the same bytes
    scale_row_bytes = k_fp8_scale.size(1) * k_fp8_scale.element_size()
    quant_block_size = head_dim * 4 // scale_row_bytes
    if head_dim % quant_block_size != 0:
        raise ValueError("head_dim must be divisible by quant_block_size")
    num_quant_blocks = head_dim // quant_block_size
    batch_size = block_table.shape[0]
    dev = k_cache.device
    assert dev.type == "cuda", "this operator has no CPU path"
    assert k_cache.dtype == torch.uint8 and k_cache.dim() == 3 and k_cache.is_contiguous()
    assert k_cache.shape[2] == head_dim + 4 * num_quant_blocks, "cache row = values + fp32 scales"
    assert k_fp8.dim() == 2 and k_fp8.element_size() == 1 and k_fp8.stride(1) == 1
    assert k_fp8_scale.dim() == 2 and k_fp8_scale.shape[0] >= num_tokens and k_fp8_scale.stride(1) == 1
    assert scale_row_bytes == 4 * num_quant_blocks, "one fp32 scale per quantisation group"
    assert block_table.dtype == torch.int32 and block_table.dim() == 2 and block_table.stride(1) == 1
    assert cu_seqlen.dtype == torch.int32 and cu_seqlen.dim() == 1 and cu_seqlen.is_contiguous()
    assert cu_seqlen.shape[0] == batch_size + 1
    for t in (k_fp8, k_fp8_scale, block_table, cu_seqlen):
        assert t.device == dev, "all tensors must be on the same device"
    if num_tokens == 0 or batch_size == 0 or num_blocks == 0:
        return
    with torch.cuda.device(dev):
        stream = torch.cuda.current_stream(dev).cuda_stream
        _native.check(
            _native.lib().dsv4_cp_gather_indexer_k_quant_cache(
                k_cache.data_ptr(), k_cache.stride(0), k_fp8.data_ptr(), k_fp8.stride(0), k_fp8_scale.data_ptr(),
                k_fp8_scale.stride(0) * k_fp8_scale.element_size(), block_table.data_ptr(), block_table.stride(0),
                cu_seqlen.data_ptr(), batch_size, num_tokens, block_size, head_dim, num_quant_blocks, stream,
            )
        )


__all__ = ["cp_gather_indexer_k_quant_cache"]
