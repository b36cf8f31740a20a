"""flaggems_vllm for NVIDIA B200: the DeepSeek-V4 attention-prologue hot path.

Keeps the import surface the reference package offers for this path
(src/flaggems_vllm/__init__.py:21-46): the operator at package level and under
`flaggems_vllm.ops`, the compatibility alias, `device`, `vendor_name`, `runtime`.
"""
import contextlib

import torch

from . import _native, ops, runtime, utils  # noqa: F401
from .ops import *  # noqa: F401,F403
from .ops import fused_deepseek_v4_qnorm_rope_kv_rope_quant_insert as _prologue

device = runtime.device.name
vendor_name = runtime.device.vendor_name

# compatibility alias kept by the reference (src/flaggems_vllm/__init__.py:37-46)
ops_deepseek_v4_qnorm_rope_kv_rope_quant_insert = _prologue
ops_inv_rope_fp8_quant = ops.fused_inv_rope_fp8_quant

# the FP8 format every quantising operator here produces (reference: ops/fused_inv_rope_fp8_quant.py:25-28)
SUPPORTED_FP8_DTYPE = torch.float8_e4m3fn



@contextlib.contextmanager
def use_gems(*_args, **_kwargs):
    """Kept for callers that wrap operator calls in `with flaggems_vllm.use_gems():` (the reference registers aten
    overrides inside it, src/flaggems_vllm/__init__.py:150-214).  This package registers nothing: its operators are
    the functions themselves, so the context changes nothing."""
    yield


__version__ = "0.1.0"
