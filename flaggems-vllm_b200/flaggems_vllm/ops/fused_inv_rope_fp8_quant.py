"""DeepSeek-V4 attention epilogue: inverse GPT-J RoPE on the rotary tail of o + FP8 group quantisation.

Drop-in for the reference operator of the same module path and name
(src/flaggems_vllm/ops/fused_inv_rope_fp8_quant.py:155-256): same arguments, assertions, output shapes,
strides and dtypes, for every geometry that passes its assertions (and has an even group size); the DeepSeek-V4
geometry (head_dim 512 = 448 + 64, groups of 128) runs on the vectorised kernel.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from .. import _native

SUPPORTED_FP8_DTYPE = torch.float8_e4m3fn


def _get_tma_aligned_size(size: int, align: int) -> int:
    return ((size + align - 1) // align) * align


def fused_inv_rope_fp8_quant(
    o: torch.Tensor,
    positions: torch.Tensor,
    cos_sin_cache: torch.Tensor,
    n_groups: int,
    heads_per_group: int,
    nope_dim: int = 448,
    rope_dim: int = 64,
    quant_group_size: int = 128,
    eps: float = 1e-10,
    dtype: Optional[torch.dtype] = None,
    tma_aligned_scales: bool = False,
) -> Tuple[torch.Tensor, torch.Tensor]:
    """
    Args:
        o: [num_tokens, num_heads, nope_dim + rope_dim] bfloat16
        positions: [num_tokens] int64
        cos_sin_cache: [max_position, rope_dim] float32, cos || sin

    Returns:
        o_fp8: [num_tokens, n_groups, heads_per_group * head_dim] float8_e4m3fn, strides (d, num_tokens*d, 1)
        o_scale: [num_tokens, n_groups, blocks] float32, or int32 with four UE8M0 bytes per head when
                 tma_aligned_scales; token-major storage padded to a multiple of 4 tokens
    """
    fp8_dtype = SUPPORTED_FP8_DTYPE if dtype is None else dtype
    assert fp8_dtype == torch.float8_e4m3fn, "only torch.float8_e4m3fn is supported"
    assert o.ndim == 3, "`o` must be [num_tokens, num_heads, head_dim]"
    assert positions.ndim == 1, "`positions` must be 1D"
    assert cos_sin_cache.ndim == 2, "`cos_sin_cache` must be 2D"
    assert o.stride(-1) == 1, "head_dim must be contiguous"
    assert positions.shape[0] == o.shape[0], "positions and o token count mismatch"

    num_tokens, num_heads, head_dim = o.shape
    assert num_heads == n_groups * heads_per_group
    assert head_dim == nope_dim + rope_dim
    assert head_dim % quant_group_size == 0
    assert nope_dim % quant_group_size == (quant_group_size - rope_dim)
    assert rope_dim % 2 == 0
    assert cos_sin_cache.shape[-1] == rope_dim
    assert cos_sin_cache.dtype == torch.float32
    # this implementation: bf16 activations, int64 positions, an even group size; the DeepSeek-V4 geometry
    # (448 + 64, groups of 128) with 16-byte aligned rows takes the vectorised kernel, any other a general one
    assert quant_group_size % 2 == 0, "the group size must be even"
    assert o.dtype == torch.bfloat16 and positions.dtype == torch.int64
    assert o.device.type == "cuda", "this operator has no CPU path"
    assert positions.device == o.device and cos_sin_cache.device == o.device
    assert positions.is_contiguous() and cos_sin_cache.stride(1) == 1

    chunks_per_head = head_dim // quant_group_size
    if tma_aligned_scales:
        assert chunks_per_head <= 4, "packed UE8M0 path currently expects at most 4 scale blocks per head"
        # with fewer than four the reference's kernel writes one int32 per head into storage sized for one per four
        # groups (:133-143 against :206-217 there): only four groups per head have a defined packed layout
        assert chunks_per_head == 4, "packed UE8M0 scales need four groups per head"

    d = heads_per_group * head_dim
    num_scale_blocks = d // quant_group_size
    tma_aligned_t = _get_tma_aligned_size(num_tokens, 4)
    if tma_aligned_scales:
        scale_inner, scale_dtype = (num_scale_blocks + 3) // 4, torch.int32
    else:
        scale_inner, scale_dtype = num_scale_blocks, torch.float32

    fp8_q = torch.empty((n_groups, num_tokens, d), dtype=fp8_dtype, device=o.device)
    scale = torch.empty(n_groups * scale_inner * tma_aligned_t, dtype=scale_dtype, device=o.device).as_strided(
        (n_groups, num_tokens, scale_inner), (scale_inner * tma_aligned_t, 1, tma_aligned_t))
    if num_tokens > 0:
        with torch.cuda.device(o.device):
            stream = torch.cuda.current_stream(o.device).cuda_stream
            _native.check(
                _native.lib().dsv4_fused_inv_rope_fp8_quant_geometry(
                    o.data_ptr(), o.stride(0), o.stride(1), positions.data_ptr(), cos_sin_cache.data_ptr(),
                    cos_sin_cache.stride(0), fp8_q.data_ptr(), scale.data_ptr(), scale_inner * tma_aligned_t, num_tokens,
                    tma_aligned_t, n_groups, heads_per_group, int(nope_dim), int(rope_dim), int(quant_group_size), float(eps),
                    1 if tma_aligned_scales else 0, stream,
                )
            )
    return fp8_q.transpose(0, 1), scale.transpose(0, 1)


__all__ = ["fused_inv_rope_fp8_quant"]
