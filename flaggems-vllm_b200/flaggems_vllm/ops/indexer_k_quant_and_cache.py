"""FP8 quantisation of the sparse-indexer keys into their paged cache.

Drop-in for the reference operator of the same module path and name
(src/flaggems_vllm/ops/indexer_k_quant_and_cache.py:103-132): same arguments and in-place effect on
`kv_cache` ([num_blocks, block_size, head_dim + 4*head_dim/quant_block_size] uint8: per block all value
bytes first, then all fp32 scales).  e4m3fn only (the NVIDIA format).
"""
from __future__ import annotations

import torch

from .. import _native


def indexer_k_quant_and_cache(k: torch.Tensor, kv_cache: torch.Tensor, slot_mapping: torch.Tensor, quant_block_size,
                              scale_fmt) -> None:
    num_blocks = kv_cache.shape[0]
    head_dim = k.shape[-1]
    num_tokens = slot_mapping.shape[0]
    block_size = kv_cache.shape[1]
    if head_dim % quant_block_size != 0:
        raise ValueError("head_dim must be divisible by quant_block_size")
    assert k.device.type == "cuda", "this operator has no CPU path"
    assert k.dim() == 2 and k.stride(1) == 1 and k.dtype in (torch.bfloat16, torch.float16)
    assert k.shape[0] >= num_tokens
    assert slot_mapping.dtype == torch.int64 and slot_mapping.dim() == 1 and slot_mapping.is_contiguous()
    assert kv_cache.dtype == torch.uint8 and kv_cache.dim() == 3 and kv_cache[0].is_contiguous()
    assert kv_cache.shape[2] == head_dim + 4 * (head_dim // quant_block_size), "cache row = values + fp32 scales"
    assert kv_cache.device == k.device and slot_mapping.device == k.device
    if num_tokens == 0 or num_blocks == 0:
        return
    with torch.cuda.device(k.device):
        stream = torch.cuda.current_stream(k.device).cuda_stream
        _native.check(
            _native.lib().dsv4_indexer_k_quant_and_cache(
                k.data_ptr(), k.stride(0), 1 if k.dtype == torch.float16 else 0, kv_cache.data_ptr(), kv_cache.stride(0),
                slot_mapping.data_ptr(), num_tokens, block_size, head_dim, int(quant_block_size),
                1 if scale_fmt == "ue8m0" else 0, stream,
            )
        )


__all__ = ["indexer_k_quant_and_cache"]
