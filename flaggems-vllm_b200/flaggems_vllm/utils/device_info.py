"""Device queries (reference: src/flaggems_vllm/utils/device_info.py:55-78)."""
from __future__ import annotations

import torch


def get_device_capability(device_id: int | None = None) -> tuple[int, int]:
    return torch.cuda.get_device_capability(device_id)


def get_sm_count(device_id: int | None = None) -> int:
    return torch.cuda.get_device_properties(device_id if device_id is not None else torch.cuda.current_device()).multi_processor_count
