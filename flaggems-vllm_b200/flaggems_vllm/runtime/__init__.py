"""The two runtime names callers and the reference's tests use (reference:
src/flaggems_vllm/runtime/__init__.py:23-84).  There is one backend - NVIDIA B200 - so
there is no vendor detection and no operator override table."""
from __future__ import annotations

import torch


class _Device:
    name = "cuda"
    vendor_name = "nvidia"
    # capability flags the reference's shared test helpers read (tests/accuracy_utils.py:26-28 there)
    support_fp64 = True
    support_bf16 = True
    support_int64 = True

    @property
    def device_count(self) -> int:
        return torch.cuda.device_count()


device = _Device()
torch_device_fn = torch.cuda

__all__ = ["device", "torch_device_fn"]
