"""Slot-addressed reader of the FP8 K cache written by the prologue.

The per-token arithmetic of the reference's `dequantize_and_gather_k_cache`
(src/flaggems_vllm/ops/deepseek_v4_attention_dequantize_and_gather_k_cache.py:86-120):
448 values `e4m3 * 2^(code-127)` rounded to bf16, then the 64 cached bf16 RoPE values.
"""
from __future__ import annotations

import torch

from .. import _native


def gather_dequant_k_cache_slots(k_cache: torch.Tensor, slots: torch.Tensor, cache_block_size: int,
                                 out: torch.Tensor | None = None) -> torch.Tensor:
    """bf16 [len(slots), 512]: the cached tokens at `slots` (a negative slot gives a zero row)."""
    assert k_cache.dtype == torch.uint8 and k_cache.dim() == 2 and k_cache.stride(1) == 1
    assert slots.dtype == torch.int64 and slots.dim() == 1 and slots.is_contiguous()
    assert k_cache.device.type == "cuda" and slots.device == k_cache.device
    assert cache_block_size > 0 and k_cache.shape[1] >= cache_block_size * 584
    n = slots.shape[0]
    if out is None:
        out = torch.empty(n, 512, dtype=torch.bfloat16, device=k_cache.device)
    assert out.dtype == torch.bfloat16 and out.shape == (n, 512) and out.stride(1) == 1 and out.device == k_cache.device
    if n == 0:
        return out
    with torch.cuda.device(k_cache.device):
        stream = torch.cuda.current_stream(k_cache.device).cuda_stream
        _native.check(
            _native.lib().dsv4_gather_dequant_k_cache(
                k_cache.data_ptr(), slots.data_ptr(), n, out.data_ptr(), out.stride(0), int(cache_block_size),
                k_cache.stride(0), stream,
            )
        )
    return out
