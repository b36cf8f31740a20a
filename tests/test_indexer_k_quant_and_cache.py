"""`indexer_k_quant_and_cache`: oracle vs vectors from the upstream test's torch statement; CUDA kernel vs both,
whole cache compared bit for bit (the upstream bar: rtol=0, atol=0)."""
from __future__ import annotations

import numpy as np
import pytest
import torch

import flaggems_vllm
from conftest import GOLDEN
from oracle import c_oracle

NAMES = sorted(p.stem for p in GOLDEN.glob("indexer_*f16_*.npz"))
DEV = "cuda:0"


def load(name):
    z = np.load(GOLDEN / f"{name}.npz")
    dtype = torch.float16 if int(z["is_fp16"]) else torch.bfloat16
    return {"k": torch.from_numpy(z["k"].view(np.int16).copy()).view(dtype), "slot_mapping": torch.from_numpy(z["slot_mapping"].copy()),
            "cache": torch.from_numpy(z["cache"].copy()), "cache_out": torch.from_numpy(z["cache_out"].copy()),
            "qbs": int(z["quant_block_size"]), "fmt": str(z["scale_fmt"])}


def test_golden_files_exist():
    assert len(NAMES) >= 5


@pytest.mark.parametrize("name", NAMES)
def test_oracle_reproduces_upstream_reference(name):
    g = load(name)
    cache = g["cache"].clone()
    c_oracle.indexer_k_quant_and_cache(g["k"], cache, g["slot_mapping"], g["qbs"], g["fmt"])
    assert torch.equal(cache, g["cache_out"])


@pytest.mark.gpu
@pytest.mark.parametrize("name", NAMES)
def test_kernel_reproduces_upstream_reference(name):
    g = load(name)
    cache = g["cache"].to(DEV)
    flaggems_vllm.indexer_k_quant_and_cache(g["k"].to(DEV), cache, g["slot_mapping"].to(DEV), g["qbs"], g["fmt"])
    assert torch.equal(cache.cpu(), g["cache_out"])


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("tokens,blocks,bs,hd,qbs,fmt", [
    (1, 2, 16, 128, 128, "ue8m0"), (1000, 40, 64, 128, 128, "ue8m0"), (333, 12, 64, 512, 128, "fp32"),
    (50, 8, 16, 256, 32, "ue8m0"), (60, 8, 12, 128, 128, "ue8m0"), (40, 8, 16, 768, 256, "ue8m0"), (30, 4, 16, 96, 48, "ue8m0"), (25, 4, 16, 120, 24, "fp32"),
])
def test_kernel_matches_oracle(dtype, tokens, blocks, bs, hd, qbs, fmt):
    """Vector path (power-of-two groups) and scalar path (48, 24), untouched slots included in the comparison."""
    g = torch.Generator().manual_seed(tokens + hd + qbs)
    k = (torch.randn(tokens, hd, generator=g) * torch.logspace(-2, 2, tokens)[:, None]).to(dtype)
    slots = torch.randperm(blocks * bs, generator=g)[:tokens].to(torch.int64)
    slots[::5] = -1
    cache = torch.randint(0, 256, (blocks, bs, hd + 4 * (hd // qbs)), generator=g, dtype=torch.uint8)
    want = cache.clone()
    c_oracle.indexer_k_quant_and_cache(k, want, slots, qbs, fmt)
    got = cache.to(DEV)
    flaggems_vllm.indexer_k_quant_and_cache(k.to(DEV), got, slots.to(DEV), qbs, fmt)
    assert torch.equal(got.cpu(), want)


def test_host_checks_without_gpu():
    k = torch.zeros(4, 128, dtype=torch.bfloat16)
    cache = torch.zeros(2, 16, 132, dtype=torch.uint8)
    slots = torch.arange(4)
    with pytest.raises(AssertionError, match="no CPU path"):
        flaggems_vllm.indexer_k_quant_and_cache(k, cache, slots, 128, "ue8m0")
    with pytest.raises(ValueError):
        flaggems_vllm.indexer_k_quant_and_cache(k, cache, slots, 100, "ue8m0")
