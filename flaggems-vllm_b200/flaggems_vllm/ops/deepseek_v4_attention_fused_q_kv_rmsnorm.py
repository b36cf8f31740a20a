"""Weighted RMSNorm of the q low-rank activations and of the latent KV in one launch.

Drop-in for the reference operator of the same module path and name
(src/flaggems_vllm/ops/deepseek_v4_attention_fused_q_kv_rmsnorm.py:65-103): same arguments,
assertions and return value.  Rows and weights may be bfloat16, float16 or float32, each tensor its own, as the
reference kernel allows; all-bfloat16 (what the DeepSeek-V4 attention layer passes) takes the vectorised kernel.
"""
from __future__ import annotations

from typing import Tuple

import torch

from .. import _native


_DTYPE_CODE = {torch.bfloat16: 0, torch.float16: 1, torch.float32: 2}


def fused_q_kv_rmsnorm(qr: torch.Tensor, kv: torch.Tensor, q_weight: torch.Tensor, kv_weight: torch.Tensor,
                       eps: float) -> Tuple[torch.Tensor, torch.Tensor]:
    """(qr_out, kv_out) with out = (x * rsqrt(mean(x^2, -1) + eps)) * weight in fp32, rounded to the row's dtype."""
    assert qr.ndim == 2 and kv.ndim == 2
    assert qr.shape[0] == kv.shape[0]
    assert qr.stride(-1) == 1 and kv.stride(-1) == 1
    assert q_weight.is_contiguous() and kv_weight.is_contiguous()
    assert qr.device.type == "cuda", "this operator has no CPU path"
    for t in (qr, kv, q_weight, kv_weight):
        assert t.dtype in _DTYPE_CODE, "bfloat16, float16 or float32"
        assert t.device == qr.device, "all tensors must be on the same device"
    assert q_weight.shape == (qr.shape[1],) and kv_weight.shape == (kv.shape[1],)

    num_tokens = qr.shape[0]
    qr_out = torch.empty_like(qr)
    kv_out = torch.empty_like(kv)
    if num_tokens == 0:
        return qr_out, kv_out
    assert qr_out.stride(-1) == 1 and kv_out.stride(-1) == 1
    with torch.cuda.device(qr.device):
        stream = torch.cuda.current_stream(qr.device).cuda_stream
        _native.check(
            _native.lib().dsv4_fused_q_kv_rmsnorm_dtypes(
                qr.data_ptr(), qr_out.data_ptr(), q_weight.data_ptr(), qr.stride(0), qr_out.stride(0), qr.shape[1],
                _DTYPE_CODE[qr.dtype], _DTYPE_CODE[q_weight.dtype],
                kv.data_ptr(), kv_out.data_ptr(), kv_weight.data_ptr(), kv.stride(0), kv_out.stride(0), kv.shape[1],
                _DTYPE_CODE[kv.dtype], _DTYPE_CODE[kv_weight.dtype], num_tokens, float(eps), stream,
            )
        )
    return qr_out, kv_out


__all__ = ["fused_q_kv_rmsnorm"]
