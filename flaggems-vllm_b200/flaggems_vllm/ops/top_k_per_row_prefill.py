"""Top-k selection over the indexer logits of a prefill step.

Drop-in for the reference operator of the same module path and name
(src/flaggems_vllm/ops/top_k_per_row_prefill.py, wrapper `top_k_per_row_prefill`): same arguments; `indices`
[num_rows, top_k] int32 is filled in place with the positions, relative to row_starts[row], of the top_k largest
logits of each row inside [row_starts[row], row_ends[row]), in any order, -1 where the range is shorter than top_k.
"""
from __future__ import annotations

import torch

from .. import _native
from .top_k_per_row_decode import _check


def top_k_per_row_prefill(logits, row_starts, row_ends, indices, num_rows, stride0, stride1, top_k) -> None:
    _check(logits, indices, num_rows, stride0, stride1, top_k)
    for t in (row_starts, row_ends):
        assert t.dtype == torch.int32 and t.dim() == 1 and t.is_contiguous() and t.shape[0] >= num_rows and t.device == logits.device
    if num_rows == 0 or top_k == 0:
        return
    with torch.cuda.device(logits.device):
        stream = torch.cuda.current_stream(logits.device).cuda_stream
        _native.check(
            _native.lib().dsv4_top_k_per_row_prefill(logits.data_ptr(), stride0, stride1, row_starts.data_ptr(), row_ends.data_ptr(),
                                                     indices.data_ptr(), num_rows, logits.shape[1], int(top_k), stream)
        )


__all__ = ["top_k_per_row_prefill"]
