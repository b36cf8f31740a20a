"""`act_quant_triton`: oracle vs vectors from the upstream test's torch statement; CUDA kernel vs both, bytes and scales
bit for bit (the upstream test allows atol 1e-2 on the de-quantised bytes)."""
from __future__ import annotations

import numpy as np
import pytest
import torch

import flaggems_vllm
from conftest import GOLDEN
from oracle import c_oracle

NAMES = sorted(p.stem for p in GOLDEN.glob("act_quant_*.npz"))
DEV = "cuda:0"


def load(name):
    z = np.load(GOLDEN / f"{name}.npz")
    return {"x": torch.from_numpy(z["x"].view(np.int16).copy()).view(torch.bfloat16), "block": int(z["block_size"]),
            "fmt": "ue8m0" if int(z["round_scale"]) else None, "bytes": torch.from_numpy(z["bytes"].copy()), "scales": torch.from_numpy(z["scales"].copy())}


def test_golden_files_exist():
    assert len(NAMES) >= 6


@pytest.mark.parametrize("name", NAMES)
def test_oracle_reproduces_upstream_reference(name):
    g = load(name)
    q, s = c_oracle.act_quant(g["x"], g["block"], g["fmt"])
    assert torch.equal(q, g["bytes"]) and torch.equal(s.view(torch.int32), g["scales"].view(torch.int32))


@pytest.mark.gpu
@pytest.mark.parametrize("name", NAMES)
def test_kernel_reproduces_upstream_reference(name):
    g = load(name)
    q, s = flaggems_vllm.act_quant_triton(g["x"].to(DEV), g["block"], g["fmt"])
    assert q.dtype == torch.float8_e4m3fn and s.shape == g["scales"].shape
    assert torch.equal(q.view(torch.uint8).cpu(), g["bytes"]) and torch.equal(s.cpu().view(torch.int32), g["scales"].view(torch.int32))


@pytest.mark.gpu
@pytest.mark.parametrize("fmt", [None, "ue8m0"])
@pytest.mark.parametrize("rows,cols,block", [(1, 128, 128), (164, 896, 64), (512, 2048, 128), (3454, 8192, 128), (40, 2048, 256), (9, 96, 48)])
def test_kernel_matches_oracle(rows, cols, block, fmt):
    """The upstream shape list (1 ... 3454 rows, 128 ... 8192 columns, blocks of 64 and 128) and blocks off the vector path."""
    g = torch.Generator().manual_seed(rows + cols + block)
    x = (torch.randn(rows, cols, generator=g) * torch.logspace(-7, 3, rows)[:, None]).to(torch.bfloat16)
    want_q, want_s = c_oracle.act_quant(x, block, fmt)
    q, s = flaggems_vllm.act_quant_triton(x.to(DEV), block, fmt)
    assert torch.equal(q.view(torch.uint8).cpu(), want_q) and torch.equal(s.cpu().view(torch.int32), want_s.view(torch.int32))


def test_host_checks_without_gpu():
    with pytest.raises(AssertionError, match="no CPU path"):
        flaggems_vllm.act_quant_triton(torch.zeros(4, 256, dtype=torch.bfloat16), 128)
    with pytest.raises(AssertionError, match="divisible"):
        flaggems_vllm.act_quant_triton(torch.zeros(4, 256, dtype=torch.bfloat16), 100)
