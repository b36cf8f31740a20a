"""`per_token_group_quant_fp8`: oracle vs vectors from the upstream test's torch statement; CUDA kernel vs both, bytes
and scales bit for bit (the upstream test allows rtol 0.15 on the bytes and fp32 closeness on the scales)."""
from __future__ import annotations

import numpy as np
import pytest
import torch

import flaggems_vllm
from conftest import GOLDEN
from oracle import c_oracle

NAMES = sorted(p.stem for p in GOLDEN.glob("group_quant_*.npz"))
DEV = "cuda:0"


def load(name):
    z = np.load(GOLDEN / f"{name}.npz")
    return {"x": torch.from_numpy(z["x"].view(np.int16).copy()).view(torch.bfloat16), "group": int(z["group_size"]), "ue8m0": bool(int(z["ue8m0"])),
            "bytes": torch.from_numpy(z["bytes"].copy()), "scales": torch.from_numpy(z["scales"].copy())}


def same_bits(a, b):
    return torch.equal(a.contiguous().view(torch.int32), b.contiguous().view(torch.int32))


def test_golden_files_exist():
    assert len(NAMES) >= 8


@pytest.mark.parametrize("name", NAMES)
def test_oracle_reproduces_upstream_reference(name):
    g = load(name)
    q, s = c_oracle.per_token_group_quant_fp8(g["x"], g["group"], scale_ue8m0=g["ue8m0"])
    assert torch.equal(q, g["bytes"]) and same_bits(s, g["scales"])


@pytest.mark.gpu
@pytest.mark.parametrize("name", NAMES)
def test_kernel_reproduces_upstream_reference(name):
    g = load(name)
    q, s = flaggems_vllm.per_token_group_quant_fp8(g["x"].to(DEV), g["group"], scale_ue8m0=g["ue8m0"])
    assert q.dtype == torch.float8_e4m3fn and s.dtype == torch.float32 and s.shape == g["scales"].shape
    assert torch.equal(q.view(torch.uint8).cpu(), g["bytes"]) and same_bits(s.cpu(), g["scales"])


@pytest.mark.gpu
@pytest.mark.parametrize("ue8m0", [False, True])
@pytest.mark.parametrize("tokens,cols,group,column_major", [
    (1, 512, 128, False), (83, 4096, 128, False), (83, 5120, 64, True), (7, 13824, 128, True), (33, 2048, 256, False), (9, 4096, 512, True),
    (5, 96, 48, False), (6, 120, 24, True),
])
def test_kernel_matches_oracle(tokens, cols, group, column_major, ue8m0):
    """The upstream shape list (7 / 83 tokens, 512 ... 13824 columns, groups of 64 ... 512), both scale layouts, group
    sizes off the vector path, rows scaled over ten decades."""
    g = torch.Generator().manual_seed(tokens + cols + group)
    x = (torch.randn(tokens, cols, generator=g) * torch.logspace(-6, 4, tokens)[:, None]).to(torch.bfloat16)
    want_q, want_s = c_oracle.per_token_group_quant_fp8(x, group, column_major_scales=column_major, scale_ue8m0=ue8m0)
    q, s = flaggems_vllm.per_token_group_quant_fp8(x.to(DEV), group, column_major_scales=column_major, scale_ue8m0=ue8m0)
    assert s.stride() == want_s.stride()
    assert torch.equal(q.view(torch.uint8).cpu(), want_q) and torch.equal(s.cpu().view(torch.int32), want_s.view(torch.int32))


@pytest.mark.gpu
def test_other_eps_row_slices_and_three_dimensions():
    g = torch.Generator().manual_seed(4)
    wide = torch.randn(40, 1024, generator=g).to(torch.bfloat16)
    x = wide[:, 256:768]  # row stride 1024, 512 columns
    want_q, want_s = c_oracle.per_token_group_quant_fp8(x, 128, eps=1e-3)
    q, s = flaggems_vllm.per_token_group_quant_fp8(wide.to(DEV)[:, 256:768], 128, eps=1e-3)  # not the default eps: IEEE division
    assert torch.equal(q.view(torch.uint8).cpu(), want_q) and same_bits(s.cpu(), want_s)
    x3 = torch.randn(4, 10, 256, generator=g).to(torch.bfloat16)
    want_q, want_s = c_oracle.per_token_group_quant_fp8(x3.view(40, 256), 64, scale_ue8m0=True)
    q, s = flaggems_vllm.per_token_group_quant_fp8(x3.to(DEV), 64, scale_ue8m0=True)
    assert q.shape == x3.shape and s.shape == (4, 10, 4)
    assert torch.equal(q.view(torch.uint8).cpu().view(40, 256), want_q) and same_bits(s.cpu().view(40, 4), want_s)


@pytest.mark.gpu
def test_agrees_with_the_epilogue_quantiser_without_rotation():
    """fused_inv_rope_fp8_quant with an identity rotation is this operator on the same values."""
    g = torch.Generator().manual_seed(5)
    o = torch.randn(16, 8, 512, generator=g).to(torch.bfloat16).to(DEV)
    table = torch.cat([torch.ones(4, 32), torch.zeros(4, 32)], dim=1).contiguous().to(DEV)
    fp8, scale = flaggems_vllm.fused_inv_rope_fp8_quant(o, torch.zeros(16, dtype=torch.int64, device=DEV), table, 2, 4, tma_aligned_scales=False)
    q, s = flaggems_vllm.per_token_group_quant_fp8(o.view(16, 8 * 512), 128)
    # the epilogue returns [tokens, groups of heads, heads_per_group * 512] (stored group-major) and scales [tokens, groups, 16]
    assert torch.equal(fp8.view(torch.uint8).reshape(16, 4096), q.view(torch.uint8))
    assert torch.equal(scale.reshape(16, 32), s)


def test_host_checks_without_gpu():
    x = torch.zeros(4, 256, dtype=torch.bfloat16)
    with pytest.raises(AssertionError, match="no CPU path"):
        flaggems_vllm.per_token_group_quant_fp8(x, 128)
    with pytest.raises(AssertionError, match="divisible"):
        flaggems_vllm.per_token_group_quant_fp8(x, 100)
