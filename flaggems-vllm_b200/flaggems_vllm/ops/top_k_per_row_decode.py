"""Top-k selection over the indexer logits of a decode step.

Drop-in for the reference operator of the same module path and name
(src/flaggems_vllm/ops/top_k_per_row_decode.py:1263-1399): same arguments; `indices` [num_rows, top_k] int32 is
filled in place with the positions of the top_k largest logits of each row inside its valid range
[0, seq_lens[row // next_n] - next_n + row % next_n + 1), in any order, -1 where the range is shorter than top_k.
"""
from __future__ import annotations

import torch

from .. import _native


def _check(logits, indices, num_rows, stride0, stride1, top_k):
    assert num_rows == logits.shape[0]
    assert logits.dim() == 2 and logits.dtype == torch.float32, "float32 logits [num_rows, vocab]"
    assert logits.device.type == "cuda", "this operator has no CPU path"
    assert stride0 == logits.stride(0) and stride1 == logits.stride(1)
    assert indices.dtype == torch.int32 and indices.dim() == 2 and indices.is_contiguous()
    assert indices.shape[0] >= num_rows and indices.shape[1] == top_k and indices.device == logits.device


def top_k_per_row_decode(logits, next_n, seq_lens, indices, num_rows, stride0, stride1, top_k) -> None:
    _check(logits, indices, num_rows, stride0, stride1, top_k)
    assert seq_lens.dtype == torch.int32 and seq_lens.dim() == 1 and seq_lens.is_contiguous() and seq_lens.device == logits.device
    assert next_n >= 1 and seq_lens.shape[0] * next_n >= num_rows
    if num_rows == 0 or top_k == 0:
        return
    with torch.cuda.device(logits.device):
        stream = torch.cuda.current_stream(logits.device).cuda_stream
        _native.check(
            _native.lib().dsv4_top_k_per_row_decode(logits.data_ptr(), stride0, stride1, int(next_n), seq_lens.data_ptr(),
                                                    indices.data_ptr(), num_rows, logits.shape[1], int(top_k), stream)
        )


__all__ = ["top_k_per_row_decode"]
