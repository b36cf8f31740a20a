"""Top-k positions inside a request -> slots of the paged cache, and per-token counts.

Drop-in for the reference operator of the same module path and name
(src/flaggems_vllm/ops/deepseek_v4_attention_compute_global_topk_indices_and_lens.py:128-161): same arguments
and return values (int32 indices shaped like `topk_indices`, int32 lens).
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from .. import _native


def compute_global_topk_indices_and_lens(
    topk_indices: torch.Tensor,
    token_to_req_indices: torch.Tensor,
    block_table: torch.Tensor,
    block_size: int,
    is_valid_token: Optional[torch.Tensor] = None,
) -> Tuple[torch.Tensor, torch.Tensor]:
    assert topk_indices.ndim == 2
    dev = topk_indices.device
    assert dev.type == "cuda", "this operator has no CPU path"
    assert topk_indices.dtype == torch.int32 and topk_indices.stride(1) == 1, "int32 indices with unit inner stride"
    assert token_to_req_indices.dtype == torch.int32 and token_to_req_indices.is_contiguous()
    assert block_table.dtype == torch.int32 and block_table.dim() == 2 and block_table.stride(1) == 1
    num_tokens, topk = topk_indices.shape
    assert token_to_req_indices.shape == (num_tokens,)
    if is_valid_token is not None:
        assert is_valid_token.dtype == torch.int32 and is_valid_token.shape == (num_tokens,) and is_valid_token.is_contiguous()
    for t in (token_to_req_indices, block_table) + (() if is_valid_token is None else (is_valid_token,)):
        assert t.device == dev, "all tensors must be on the same device"
    assert int(block_size) > 0
    global_indices = torch.empty_like(topk_indices, dtype=torch.int32)
    lens = torch.empty((num_tokens,), device=dev, dtype=torch.int32)
    if num_tokens == 0:
        return global_indices, lens
    with torch.cuda.device(dev):
        stream = torch.cuda.current_stream(dev).cuda_stream
        _native.check(
            _native.lib().dsv4_compute_global_topk_indices_and_lens(
                topk_indices.data_ptr(), topk_indices.stride(0), token_to_req_indices.data_ptr(), block_table.data_ptr(),
                block_table.stride(0), None if is_valid_token is None else is_valid_token.data_ptr(),
                global_indices.data_ptr(), global_indices.stride(0), lens.data_ptr(), num_tokens, topk, int(block_size), stream,
            )
        )
    return global_indices, lens


__all__ = ["compute_global_topk_indices_and_lens"]
