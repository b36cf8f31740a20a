"""DeepSeek-V4 attention prologue: q RMSNorm + RoPE, KV RoPE + FP8 quantisation + paged insert.

Drop-in for the reference operator of the same module path and name
(src/flaggems_vllm/ops/fused_deepseek_v4_qnorm_rope_kv_rope_quant_insert.py:289-351):
same positional arguments, dtypes, shapes, in-place effects and `AssertionError`s.
The work is one hand-written sm_100a CUDA kernel reached through the C ABI of
libdsv4_prologue.so; there is no Triton, no vendor dispatch and no CPU fallback.
"""
from __future__ import annotations

import torch

from .. import _native

HEAD_DIM = 512
ROPE_DIM = 64
TOKEN_BYTES = 584  # 448 e4m3 + 64 bf16 + 8 scale bytes per cached token


def _check_arguments(q, kv, k_cache, slot_mapping, position_ids, cos_sin_cache, cache_block_size):
    """The reference's checks (:320-333) in its order and with its exception type, then what the reference leaves
    to chance and a raw-pointer kernel cannot.  Returns (num_tokens, num_heads, num_tokens_insert, device index).
    Written for a short call: decode-sized launches run about as long as this function."""
    assert q.is_contiguous() and kv.is_contiguous()
    num_tokens, num_heads, head_dims = q.shape
    assert head_dims == HEAD_DIM
    assert kv.shape == (num_tokens, HEAD_DIM)
    assert q.dtype == torch.bfloat16 and kv.dtype == torch.bfloat16
    assert k_cache.dtype == torch.uint8
    assert slot_mapping.dim() == 1
    num_tokens_insert = slot_mapping.shape[0]
    assert num_tokens_insert <= num_tokens
    assert slot_mapping.dtype == torch.int64
    assert position_ids.shape == (num_tokens,)
    assert position_ids.dtype == torch.int64
    assert cos_sin_cache.dim() == 2 and cos_sin_cache.shape[1] == ROPE_DIM
    assert cos_sin_cache.dtype == torch.float32
    assert k_cache.dim() == 2 and k_cache.stride(1) == 1, "k_cache must be [num_blocks, block_bytes] with unit byte stride"
    assert cache_block_size > 0 and k_cache.shape[1] >= cache_block_size * TOKEN_BYTES, "cache block too small"
    assert slot_mapping.is_contiguous() and position_ids.is_contiguous() and cos_sin_cache.is_contiguous()
    index = q.get_device()  # -1 for a CPU tensor
    assert index >= 0 and q.is_cuda, "this operator has no CPU path: tensors must live on a CUDA device"
    assert (kv.get_device() == index and k_cache.get_device() == index and slot_mapping.get_device() == index
            and position_ids.get_device() == index and cos_sin_cache.get_device() == index), "all tensors must be on the same device"
    return num_tokens, num_heads, num_tokens_insert, index


# raw handle of the current stream without building a torch.cuda.Stream object
_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None) or (lambda index: torch.cuda.current_stream(index).cuda_stream)
_launch = None  # the bound C entry point, looked up once


def _bind():
    global _launch
    _launch = _native.lib().dsv4_qnorm_rope_kv_insert
    return _launch


def fused_deepseek_v4_qnorm_rope_kv_rope_quant_insert(
    q: torch.Tensor,
    kv: torch.Tensor,
    k_cache: torch.Tensor,
    slot_mapping: torch.Tensor,
    position_ids: torch.Tensor,
    cos_sin_cache: torch.Tensor,
    eps: float,
    cache_block_size: int,
) -> None:
    """Per-head weight-less RMSNorm + GPT-J RoPE for q (in place), and GPT-J RoPE + UE8M0
    FP8 quantisation + paged-cache insertion for the latent KV, in one kernel launch on
    the current stream of q's device.

    K-cache block layout (reference docstring, :303-308): `cache_block_size` token records
    of 576 bytes (448 e4m3 bytes + 64 bf16), then `cache_block_size` groups of 8 scale
    bytes (7 UE8M0 codes + 1 zero); `k_cache.stride(0)` is the block pitch.

    Args:
        q: [num_tokens, num_heads, 512] bfloat16, contiguous, modified in place
        kv: [num_tokens, 512] bfloat16, contiguous, read only
        k_cache: [num_blocks, block_bytes] uint8, modified in place at the mapped slots
        slot_mapping: [num_tokens_insert <= num_tokens] int64; negative entries are skipped
        position_ids: [num_tokens] int64
        cos_sin_cache: [max_pos, 64] float32 (32 cos | 32 sin)
        eps: RMSNorm epsilon
        cache_block_size: tokens per cache block
    """
    num_tokens, num_heads, num_tokens_insert, index = _check_arguments(
        q, kv, k_cache, slot_mapping, position_ids, cos_sin_cache, cache_block_size)
    if num_tokens == 0:
        return
    launch = _launch or _bind()
    # the library launches on the current device: switch only when q lives elsewhere (the guard costs
    # several microseconds, which matters for decode-sized calls outside CUDA graphs)
    if index == torch.cuda.current_device():
        code = launch(q.data_ptr(), kv.data_ptr(), k_cache.data_ptr(), slot_mapping.data_ptr(), position_ids.data_ptr(),
                      cos_sin_cache.data_ptr(), float(eps), num_tokens, num_heads, num_tokens_insert, int(cache_block_size),
                      k_cache.stride(0), _raw_stream(index))
    else:
        with torch.cuda.device(index):
            code = launch(q.data_ptr(), kv.data_ptr(), k_cache.data_ptr(), slot_mapping.data_ptr(), position_ids.data_ptr(),
                          cos_sin_cache.data_ptr(), float(eps), num_tokens, num_heads, num_tokens_insert, int(cache_block_size),
                          k_cache.stride(0), _raw_stream(index))
    if code != 0:
        _native.check(code)


def fused_deepseek_v4_qnorm_rope_kv_rope_quant_insert_padded(
    q: torch.Tensor,
    kv: torch.Tensor,
    k_cache: torch.Tensor,
    slot_mapping: torch.Tensor,
    position_ids: torch.Tensor,
    cos_sin_cache: torch.Tensor,
    padded_heads: int,
    eps: float,
    cache_block_size: int,
) -> torch.Tensor:
    """The nine-argument, out-of-place form vLLM >= 0.22 uses: q is left untouched and a new tensor
    [num_tokens, padded_heads, 512] is returned whose first num_heads heads hold the normalised, rotated q and
    whose remaining heads are zero; the KV side is the same as in the in-place operator."""
    num_tokens, num_heads, num_tokens_insert, _ = _check_arguments(
        q, kv, k_cache, slot_mapping, position_ids, cos_sin_cache, cache_block_size)
    dev = q.device
    assert padded_heads >= num_heads
    q_out = torch.empty(num_tokens, padded_heads, HEAD_DIM, dtype=q.dtype, device=dev)
    if num_tokens == 0:
        return q_out
    with torch.cuda.device(dev):
        stream = torch.cuda.current_stream(dev).cuda_stream
        _native.check(
            _native.lib().dsv4_qnorm_rope_kv_insert_padded(
                q.data_ptr(), q_out.data_ptr(), kv.data_ptr(), k_cache.data_ptr(), slot_mapping.data_ptr(),
                position_ids.data_ptr(), cos_sin_cache.data_ptr(), float(eps), num_tokens, num_heads, int(padded_heads),
                num_tokens_insert, int(cache_block_size), k_cache.stride(0), stream,
            )
        )
    return q_out


def fused_deepseek_v4_qnorm_rope_kv_rope_quant_insert_checked(
    q, kv, k_cache, slot_mapping, position_ids, cos_sin_cache, eps, cache_block_size
) -> int:
    """Debug form: same effects, but positions outside the table and slots outside the cache
    are skipped on the device and reported.  Returns a bit mask (bit 0: a bad position, bit 1:
    a bad slot); 0 means every index was in range.  Synchronises to read the mask."""
    num_tokens, num_heads, num_tokens_insert, _ = _check_arguments(
        q, kv, k_cache, slot_mapping, position_ids, cos_sin_cache, cache_block_size)
    status = torch.zeros(1, dtype=torch.int32, device=q.device)
    if num_tokens == 0:
        return 0
    lib = _native.lib()
    with torch.cuda.device(q.device):
        stream = torch.cuda.current_stream(q.device).cuda_stream
        _native.check(
            lib.dsv4_qnorm_rope_kv_insert_checked(
                q.data_ptr(), kv.data_ptr(), k_cache.data_ptr(), slot_mapping.data_ptr(), position_ids.data_ptr(),
                cos_sin_cache.data_ptr(), float(eps), num_tokens, num_heads, num_tokens_insert,
                int(cache_block_size), k_cache.stride(0), k_cache.shape[0], cos_sin_cache.shape[0],
                status.data_ptr(), stream,
            )
        )
    return int(status.item())
