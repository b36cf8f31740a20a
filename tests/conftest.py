"""pytest configuration: import paths, the `gpu` marker, golden-vector loading."""
from __future__ import annotations

import sys
from pathlib import Path

import numpy as np
import pytest
import torch

ROOT = Path(__file__).resolve().parent.parent
for p in (ROOT, ROOT / "flaggems-vllm_b200"):
    if str(p) not in sys.path:
        sys.path.insert(0, str(p))

GOLDEN = Path(__file__).resolve().parent / "golden"
SMALL_GOLDEN_CASES = ("q_path", "kv_path_bs16", "kv_path_bs64", "dp_padding", "mixed", "edge_rows", "padded_stride")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")
    # rebuild the CUDA library when a source is newer than it (no-op otherwise; nvcc cross-compiles)
    from flaggems_vllm import build as native_build

    native_build.build()


def pytest_collection_modifyitems(config, items):
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


def _bf16(a: np.ndarray) -> torch.Tensor:
    return torch.from_numpy(a.view(np.int16).copy()).view(torch.bfloat16)


def load_golden(name: str) -> dict:
    """A stored case as torch CPU tensors: inputs, the upstream reference's outputs, scalars."""
    z = np.load(GOLDEN / f"{name}.npz")
    from flaggems_vllm.testing.workloads import cos_sin_table

    return {
        "q": _bf16(z["q"]), "kv": _bf16(z["kv"]), "k_cache": torch.from_numpy(z["k_cache"].copy()),
        "slot_mapping": torch.from_numpy(z["slot_mapping"].copy()),
        "position_ids": torch.from_numpy(z["position_ids"].copy()),
        "cos_sin_cache": cos_sin_table(int(z["max_pos"])), "eps": float(z["eps"]), "block_size": int(z["block_size"]),
        "q_out": _bf16(z["q_out"]), "k_cache_out": torch.from_numpy(z["k_cache_out"].copy()),
    }


@pytest.fixture(params=SMALL_GOLDEN_CASES)
def golden_case(request):
    return request.param, load_golden(request.param)
