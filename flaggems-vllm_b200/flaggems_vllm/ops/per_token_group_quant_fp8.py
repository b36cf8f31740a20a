"""FP8 e4m3 quantisation of activations in groups along the last dimension, one fp32 scale per group.

Drop-in for the reference operator of the same module path and name
(src/flaggems_vllm/ops/per_token_group_quant_fp8.py:226-330): same arguments and return values (x_q shaped like x,
scales [..., K / group_size] float32, transposed storage when `column_major_scales`).  bfloat16 inputs and
float8_e4m3fn outputs (the NVIDIA format) only.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from .. import _native

SUPPORTED_FP8_DTYPE = torch.float8_e4m3fn


def per_token_group_quant_fp8(
    x: torch.Tensor,
    group_size: int,
    eps: float = 1e-10,
    dtype: Optional[torch.dtype] = None,
    column_major_scales: bool = False,
    scale_ue8m0: bool = False,
) -> Tuple[torch.Tensor, torch.Tensor]:
    fp8_dtype = SUPPORTED_FP8_DTYPE if dtype is None else dtype
    assert x.shape[-1] % group_size == 0, (
        f"the last dimension of `x` {x.shape[-1]} must be divisible by `group_size` {group_size}")
    assert x.stride(-1) == 1, "`x` groups must be contiguous"
    assert x.device.type == "cuda", "this operator has no CPU path"
    assert x.dtype == torch.bfloat16 and fp8_dtype == torch.float8_e4m3fn, "bfloat16 -> float8_e4m3fn only"
    assert x.dim() >= 2 and (x.dim() == 2 or x.is_contiguous()), "[M, K] with any row stride, or a contiguous tensor of more dimensions"
    cols = x.shape[-1]
    x2 = x if x.dim() == 2 else x.view(-1, cols)
    rows = x2.shape[0]
    x_q = torch.empty(x.shape, device=x.device, dtype=fp8_dtype)
    if column_major_scales:
        shape = (cols // group_size,) + x.shape[:-1]
        x_s = torch.empty(shape, device=x.device, dtype=torch.float32).permute(-1, -2)
        assert x.dim() == 2, "column-major scales for [M, K] inputs"
        stride_row, stride_group = x_s.stride(0), x_s.stride(1)
    else:
        x_s = torch.empty(x.shape[:-1] + (cols // group_size,), device=x.device, dtype=torch.float32)
        stride_row, stride_group = cols // group_size, 1
    if rows == 0 or cols == 0:
        return x_q, x_s
    with torch.cuda.device(x.device):
        stream = torch.cuda.current_stream(x.device).cuda_stream
        _native.check(
            _native.lib().dsv4_per_token_group_quant_fp8(x2.data_ptr(), x2.stride(0), x_q.data_ptr(), x_s.data_ptr(), stride_row, stride_group,
                                                         rows, cols, int(group_size), float(eps), 1 if scale_ue8m0 else 0, stream)
        )
    return x_q, x_s


__all__ = ["per_token_group_quant_fp8"]
