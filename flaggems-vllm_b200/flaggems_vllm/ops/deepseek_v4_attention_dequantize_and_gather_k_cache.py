"""Reader of the DeepSeek-V4 FP8 K cache: gather tokens through a block table and de-quantise them.

Drop-in for the reference operator of the same module path and name
(src/flaggems_vllm/ops/deepseek_v4_attention_dequantize_and_gather_k_cache.py:123-172): same arguments,
same assertions, `out` filled in place.  One CUDA kernel through the C ABI; no Triton, no fallback.
"""
from __future__ import annotations

from typing import Optional

import torch

from .. import _native


def _default_scale_slots(nope_dim: int) -> int:
    return (nope_dim + 63) // 64 + (1 if nope_dim % 64 == 0 else 0)


def _as_cache_2d(k_cache: torch.Tensor) -> torch.Tensor:
    if k_cache.ndim == 2:
        return k_cache
    if k_cache.ndim == 3:
        return (k_cache if k_cache.is_contiguous() else k_cache.contiguous()).view(k_cache.shape[0], -1)
    raise ValueError(f"k_cache must be 2D or 3D, got shape={tuple(k_cache.shape)}")


def dequantize_and_gather_k_cache(
    out: torch.Tensor,
    k_cache: torch.Tensor,
    seq_lens: torch.Tensor,
    gather_lens: Optional[torch.Tensor],
    block_table: torch.Tensor,
    block_size: int,
    offset: int = 0,
    rope_dim: int = 64,
    nope_dim: Optional[int] = None,
    scale_slots: Optional[int] = None,
) -> None:
    """out[r, offset + i, :nope_dim + rope_dim] = token at position seq_lens[r] - gather_lens[r] + i of
    request r (the whole sequence when gather_lens is None), read from the paged cache through
    block_table[r] and de-quantised: e4m3 * 2^(scale byte - 127) per 64 values -> bf16, RoPE bf16 copied."""
    assert out.ndim == 3 and out.dtype == torch.bfloat16
    assert seq_lens.ndim == 1 and block_table.ndim == 2
    assert seq_lens.shape[0] == block_table.shape[0] <= out.shape[0]
    output_dim = out.shape[-1]
    if nope_dim is None:
        nope_dim = output_dim - rope_dim
    if scale_slots is None:
        scale_slots = _default_scale_slots(nope_dim)
    assert nope_dim + rope_dim <= output_dim
    k_cache_2d = _as_cache_2d(k_cache)
    # what a raw-pointer kernel additionally needs
    assert out.device.type == "cuda", "this operator has no CPU path"
    assert k_cache_2d.dtype == torch.uint8 and k_cache_2d.stride(1) == 1 and out.stride(2) == 1
    index_dtype = seq_lens.dtype
    assert index_dtype in (torch.int32, torch.int64) and block_table.dtype == index_dtype
    assert seq_lens.is_contiguous() and block_table.is_contiguous()
    if gather_lens is not None:
        assert gather_lens.dtype == index_dtype and gather_lens.is_contiguous() and gather_lens.shape == seq_lens.shape
    for t in (k_cache_2d, seq_lens, block_table) + ((gather_lens,) if gather_lens is not None else ()):
        assert t.device == out.device, "all tensors must be on the same device"
    num_reqs = seq_lens.shape[0]
    if num_reqs == 0 or out.shape[1] == 0:
        return
    with torch.cuda.device(out.device):
        stream = torch.cuda.current_stream(out.device).cuda_stream
        _native.check(
            _native.lib().dsv4_dequantize_and_gather_k_cache(
                out.data_ptr(), out.stride(0), out.stride(1), out.shape[1], k_cache_2d.data_ptr(), seq_lens.data_ptr(),
                gather_lens.data_ptr() if gather_lens is not None else None, block_table.data_ptr(), num_reqs,
                block_table.shape[1], int(block_size), k_cache_2d.stride(0), int(offset), int(nope_dim), int(rope_dim),
                int(scale_slots), 1 if index_dtype == torch.int64 else 0, stream,
            )
        )


__all__ = ["dequantize_and_gather_k_cache"]
