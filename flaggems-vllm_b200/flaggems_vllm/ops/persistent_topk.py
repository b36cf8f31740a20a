"""Top-k selection over the indexer logits of a decode step, vLLM's `persistent_topk` call shape.

Drop-in for the reference operator of the same module path and name
(src/flaggems_vllm/ops/persistent_topk.py:2179-2342): same arguments and assertions; `output` [num_rows, k] int32 is
filled in place with the positions of the k largest logits of each row inside [0, lengths[row]), in any order, -1
where the row is shorter than k.  `workspace` is accepted for call compatibility and left untouched: the reference
keeps cross-CTA histograms and arrival counters there, this kernel keeps its state in shared memory (a thread-block
cluster shares a long row through distributed shared memory), so there is nothing to zero between calls.
"""
from __future__ import annotations

import torch

from .. import _native


def persistent_topk(logits: torch.Tensor, lengths: torch.Tensor, output: torch.Tensor, workspace: torch.Tensor, k: int = 512,
                    max_seq_len: int | None = None) -> None:
    assert logits.is_cuda, "persistent_topk: logits must be CUDA tensor"
    assert lengths.is_cuda, "persistent_topk: lengths must be CUDA tensor"
    assert output.is_cuda, "persistent_topk: output must be CUDA tensor"
    assert logits.dtype == torch.float32, "persistent_topk: only float32 supported"
    assert lengths.dtype == torch.int32, "persistent_topk: lengths must be int32"
    assert output.dtype == torch.int32, "persistent_topk: output must be int32"
    assert logits.dim() == 2, "persistent_topk: logits must be 2D"
    assert lengths.dim() in (1, 2), "persistent_topk: lengths must be 1D or 2D"
    assert lengths.is_contiguous(), "persistent_topk: lengths must be contiguous"
    assert output.dim() == 2, "persistent_topk: output must be 2D"
    num_rows = logits.size(0)
    seq_lens = lengths.reshape(-1) if lengths.dim() == 2 else lengths
    assert seq_lens.numel() == num_rows, f"persistent_topk: lengths size mismatch: {seq_lens.numel()} vs {num_rows}"
    assert output.size(0) == num_rows and output.size(1) == k, (
        f"persistent_topk: output size mismatch: ({output.size(0)}, {output.size(1)}) vs ({num_rows}, {k})")
    assert k in (512, 1024, 2048), f"persistent_topk supports k=512, k=1024, or k=2048, got k={k}"
    assert output.is_contiguous() and logits.device == output.device == lengths.device
    if num_rows == 0:
        return
    # a row never reaches beyond max_seq_len (the reference sizes its chunks by it)
    width = logits.shape[1] if max_seq_len is None else min(logits.shape[1], int(max_seq_len))
    with torch.cuda.device(logits.device):
        stream = torch.cuda.current_stream(logits.device).cuda_stream
        _native.check(
            _native.lib().dsv4_top_k_per_row_prefill(logits.data_ptr(), logits.stride(0), logits.stride(1), None, seq_lens.data_ptr(),
                                                     output.data_ptr(), num_rows, width, int(k), stream)
        )


__all__ = ["persistent_topk"]
