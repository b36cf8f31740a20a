"""Block-wise FP8 activation quantisation (DeepSeek's `act_quant`).

Drop-in for the reference operator of the same module path and name
(src/flaggems_vllm/ops/act_quant.py:113-175): same arguments and return values (float8_e4m3fn tensor shaped like x,
float32 scales [..., N / block_size]).  bfloat16 inputs only.  The name keeps the reference's `_triton` suffix because
that is what callers import; nothing here is Triton.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from .. import _native


def act_quant_triton(x: torch.Tensor, block_size: int = 128, scale_fmt: Optional[str] = None) -> Tuple[torch.Tensor, torch.Tensor]:
    assert x.is_contiguous(), "Input tensor must be contiguous"
    assert x.size(-1) % block_size == 0, f"Last dimension size must be divisible by block_size (block_size={block_size})"
    assert x.device.type == "cuda", "this operator has no CPU path"
    assert x.dtype == torch.bfloat16, "bfloat16 only"
    n = x.size(-1)
    x_2d = x.view(-1, n)
    m = x_2d.size(0)
    y = torch.empty_like(x, dtype=torch.float8_e4m3fn)
    s = x.new_empty(*x.size()[:-1], n // block_size, dtype=torch.float32)
    if m == 0 or n == 0:
        return y, s
    with torch.cuda.device(x.device):
        stream = torch.cuda.current_stream(x.device).cuda_stream
        _native.check(
            _native.lib().dsv4_act_quant(x_2d.data_ptr(), x_2d.stride(0), y.data_ptr(), s.data_ptr(), m, n, int(block_size),
                                         1 if scale_fmt is not None else 0, stream)
        )
    return y, s


__all__ = ["act_quant_triton"]
