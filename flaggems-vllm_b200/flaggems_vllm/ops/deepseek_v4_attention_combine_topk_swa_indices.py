"""Rows [compressed top-k entries | sliding-window entries | -1 padding] of indices into the gathered key buffer.

Drop-in for the reference operator of the same module path and name
(src/flaggems_vllm/ops/deepseek_v4_attention_combine_topk_swa_indices.py:109-161): same arguments and return
values (int32 [num_tokens, round_up(topk + window_size, 128)] and int32 lens).  Rows of tokens that no request
covers are left uninitialised, as in the reference.
"""
from __future__ import annotations

from typing import Tuple

import torch

from .. import _native

_SPARSE_PREFILL_TOPK_ALIGNMENT = 128


def combine_topk_swa_indices(
    topk_indices: torch.Tensor,
    query_start_loc: torch.Tensor,
    seq_lens: torch.Tensor,
    gather_lens: torch.Tensor,
    window_size: int,
    compress_ratio: int,
    topk: int,
    M: int,
    N: int,
) -> Tuple[torch.Tensor, torch.Tensor]:
    assert topk_indices.ndim == 2
    dev = topk_indices.device
    assert dev.type == "cuda", "this operator has no CPU path"
    num_tokens = topk_indices.shape[0]
    num_reqs = seq_lens.shape[0]
    assert topk_indices.dtype == torch.int32 and topk_indices.stride(1) == 1, "int32 indices with unit inner stride"
    assert topk <= topk_indices.shape[1], "topk entries are read from every row"
    for t in (query_start_loc, seq_lens, gather_lens):
        assert t.dtype == torch.int32 and t.dim() == 1 and t.is_contiguous() and t.device == dev
    assert query_start_loc.shape[0] >= num_reqs + 1 and gather_lens.shape[0] >= num_reqs
    combined_topk = (
        (topk + window_size + _SPARSE_PREFILL_TOPK_ALIGNMENT - 1) // _SPARSE_PREFILL_TOPK_ALIGNMENT * _SPARSE_PREFILL_TOPK_ALIGNMENT
    )
    combined = torch.empty((num_tokens, combined_topk), device=dev, dtype=torch.int32)
    lens = torch.empty((num_tokens,), device=dev, dtype=torch.int32)
    if num_tokens == 0 or num_reqs == 0:
        return combined, lens
    with torch.cuda.device(dev):
        stream = torch.cuda.current_stream(dev).cuda_stream
        _native.check(
            _native.lib().dsv4_combine_topk_swa_indices(
                topk_indices.data_ptr(), topk_indices.stride(0), topk_indices.shape[1], query_start_loc.data_ptr(),
                seq_lens.data_ptr(), gather_lens.data_ptr(), combined.data_ptr(), combined.stride(0), combined_topk,
                lens.data_ptr(), num_reqs, num_tokens, int(window_size), int(compress_ratio), int(topk), int(M), int(N), stream,
            )
        )
    return combined, lens


__all__ = ["combine_topk_swa_indices"]
