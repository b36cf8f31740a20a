"""Sparse-indexer prologue: GPT-J RoPE on the index-q tail + FP8 (per head) or MXFP4 (per 32) quantisation.

Drop-in for the reference operator of the same module path and name
(src/flaggems_vllm/ops/fused_indexer_q_rope_quant.py:283-410): same arguments, return structure, dtypes
and weight-fold semantics.  bf16 index_q, head_dim 64 / 128 / 256.
"""
from __future__ import annotations

import torch

from .. import _native

MXFP4_BLOCK_SIZE = 32
_WEIGHT_DTYPES = {torch.bfloat16: 0, torch.float16: 1, torch.float32: 2}


def fused_indexer_q_rope_quant(
    positions: torch.Tensor,
    index_q: torch.Tensor,
    index_q_cos_sin_cache: torch.Tensor,
    index_weights: torch.Tensor,
    index_weights_softmax_scale: float,
    index_weights_head_scale: float,
    use_fp4: bool = False,
):
    """Returns (q_quant, weights_out).

    FP8 (default): q_quant float8_e4m3fn like index_q, one power-of-two scale per (token, head) that is
    folded into weights_out = weights * q_scale * softmax_scale * head_scale.
    MXFP4: q_quant = (uint8 [T, H, D/2] with two e2m1 codes per byte, int32 [T, H] holding the four UE8M0
    block-scale bytes when D = 128, else uint8 [T, H, D/32] viewed as int32); weights_out = weights *
    softmax_scale * head_scale.
    """
    assert positions.ndim == 1
    assert index_q.ndim == 3
    assert index_q_cos_sin_cache.ndim == 2
    num_tokens = positions.shape[0]
    num_heads, head_dim = index_q.shape[1], index_q.shape[2]
    rot_dim = index_q_cos_sin_cache.shape[-1]

    if use_fp4 and not index_q.is_cuda:
        raise RuntimeError("MXFP4 fused_indexer_q_rope_quant requires CUDA")
    assert index_q.device.type == "cuda", "this operator has no CPU path"
    assert index_q.dtype == torch.bfloat16 and index_q.stride(2) == 1 and index_q.shape[0] == num_tokens
    assert positions.dtype == torch.int64 and positions.is_contiguous()
    assert index_q_cos_sin_cache.dtype in (torch.float32, torch.bfloat16) and index_q_cos_sin_cache.stride(1) == 1
    assert index_weights.dtype in _WEIGHT_DTYPES and index_weights.shape == (num_tokens, num_heads)
    assert index_weights.stride(1) == 1
    assert head_dim in (64, 128, 256), "head_dim must be 64, 128 or 256"
    assert rot_dim % 2 == 0 and rot_dim <= head_dim and (head_dim - rot_dim) % (head_dim // 32) == 0
    for t in (positions, index_q_cos_sin_cache, index_weights):
        assert t.device == index_q.device, "all tensors must be on the same device"

    index_weights_out = torch.empty_like(index_weights, dtype=torch.float32)
    assert index_weights_out.stride(1) == 1 or num_heads == 1
    if use_fp4:
        assert head_dim % MXFP4_BLOCK_SIZE == 0
        q_out = torch.empty((num_tokens, num_heads, head_dim // 2), dtype=torch.uint8, device=index_q.device)
        q_scale = torch.empty((num_tokens, num_heads, head_dim // MXFP4_BLOCK_SIZE), dtype=torch.uint8, device=index_q.device)
        scale_args = (q_scale.data_ptr(), q_scale.stride(0), q_scale.stride(1))
    else:
        q_out = torch.empty_like(index_q, dtype=torch.float8_e4m3fn)
        assert q_out.stride(2) == 1
        q_scale = None
        scale_args = (None, 0, 0)
    if num_tokens > 0:
        with torch.cuda.device(index_q.device):
            stream = torch.cuda.current_stream(index_q.device).cuda_stream
            _native.check(
                _native.lib().dsv4_fused_indexer_q_rope_quant(
                    positions.data_ptr(), index_q.data_ptr(), index_q.stride(0), index_q.stride(1),
                    index_q_cos_sin_cache.data_ptr(), index_q_cos_sin_cache.stride(0),
                    1 if index_q_cos_sin_cache.dtype == torch.bfloat16 else 0, rot_dim, q_out.data_ptr(), q_out.stride(0),
                    q_out.stride(1), *scale_args, index_weights.data_ptr(), index_weights.stride(0),
                    _WEIGHT_DTYPES[index_weights.dtype], index_weights_out.data_ptr(), index_weights_out.stride(0),
                    float(index_weights_softmax_scale), float(index_weights_head_scale), num_tokens, num_heads, head_dim,
                    1 if use_fp4 else 0, stream,
                )
            )
    if use_fp4:
        # four UE8M0 bytes per head (head_dim 128) are handed on as one int32, as the reference does; other
        # head sizes keep the byte tensor where the reference's int32 view is only defined for multiples of 4
        if q_scale.shape[-1] % 4 == 0:
            q_scale = q_scale.view(torch.int32).squeeze(-1)
        return (q_out, q_scale), index_weights_out
    return q_out, index_weights_out


__all__ = ["fused_indexer_q_rope_quant"]
