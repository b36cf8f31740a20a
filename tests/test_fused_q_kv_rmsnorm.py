"""`fused_q_kv_rmsnorm`: oracle vs vectors from the upstream test's torch reference; CUDA kernel vs both."""
from __future__ import annotations

import numpy as np
import pytest
import torch

import flaggems_vllm
from conftest import GOLDEN, _bf16
from flaggems_vllm.testing import compare
from oracle import c_oracle

NAMES = sorted(p.stem for p in GOLDEN.glob("rmsnorm_*.npz"))
DEV = "cuda:0"


def load(name):
    z = np.load(GOLDEN / f"{name}.npz")
    return {k: _bf16(z[k]) for k in ("qr", "kv", "q_weight", "kv_weight", "q_out", "kv_out")} | {"eps": float(z["eps"])}


def assert_within_one_ulp(a, b, max_fraction=2e-3):
    d = compare.bf16_ulp_distance(a, b)
    assert int(d.max()) <= 1, f"{int(d.max())} bf16 ulp"
    assert float((d != 0).float().mean()) <= max_fraction


@pytest.mark.parametrize("name", NAMES)
def test_oracle_matches_upstream_reference(name):
    g = load(name)
    assert_within_one_ulp(c_oracle.weighted_rmsnorm(g["qr"], g["q_weight"], g["eps"]), g["q_out"])
    assert_within_one_ulp(c_oracle.weighted_rmsnorm(g["kv"], g["kv_weight"], g["eps"]), g["kv_out"])


@pytest.mark.gpu
@pytest.mark.parametrize("name", NAMES)
def test_kernel_matches_upstream_reference(name):
    g = load(name)
    q_out, kv_out = flaggems_vllm.fused_q_kv_rmsnorm(g["qr"].to(DEV), g["kv"].to(DEV), g["q_weight"].to(DEV),
                                                     g["kv_weight"].to(DEV), g["eps"])
    assert_within_one_ulp(q_out.cpu(), g["q_out"])
    assert_within_one_ulp(kv_out.cpu(), g["kv_out"])


@pytest.mark.gpu
@pytest.mark.parametrize("tokens,qdim,kvdim", [(1, 1536, 512), (1000, 1536, 512), (17, 2048, 8), (5, 4096, 520), (9, 100, 36),
                                               (8192, 1536, 512)])
def test_kernel_matches_oracle(tokens, qdim, kvdim):
    """Sizes on the register path, beyond it (4096), and not multiples of 8 (scalar path)."""
    g = torch.Generator().manual_seed(tokens + qdim)
    qr = torch.randn(tokens, qdim, generator=g).to(torch.bfloat16)
    kv = torch.randn(tokens, kvdim, generator=g).to(torch.bfloat16)
    qw = torch.randn(qdim, generator=g).to(torch.bfloat16)
    kw = torch.randn(kvdim, generator=g).to(torch.bfloat16)
    q_in, kv_in = qr.to(DEV), kv.to(DEV)
    q_out, kv_out = flaggems_vllm.fused_q_kv_rmsnorm(q_in, kv_in, qw.to(DEV), kw.to(DEV), 1e-6)
    assert torch.equal(q_in.cpu(), qr) and torch.equal(kv_in.cpu(), kv), "inputs are read-only"
    assert_within_one_ulp(q_out.cpu(), c_oracle.weighted_rmsnorm(qr, qw, 1e-6))
    assert_within_one_ulp(kv_out.cpu(), c_oracle.weighted_rmsnorm(kv, kw, 1e-6))


@pytest.mark.gpu
def test_strided_rows():
    """qr and kv as column slices of one projection output (row stride larger than the row)."""
    g = torch.Generator().manual_seed(5)
    fused = torch.randn(64, 1536 + 512 + 64, generator=g).to(torch.bfloat16)
    qw, kw = torch.randn(1536, generator=g).to(torch.bfloat16), torch.randn(512, generator=g).to(torch.bfloat16)
    d = fused.to(DEV)
    q_out, kv_out = flaggems_vllm.fused_q_kv_rmsnorm(d[:, :1536], d[:, 1536:2048], qw.to(DEV), kw.to(DEV), 1e-6)
    assert_within_one_ulp(q_out.cpu(), c_oracle.weighted_rmsnorm(fused[:, :1536], qw, 1e-6))
    assert_within_one_ulp(kv_out.cpu(), c_oracle.weighted_rmsnorm(fused[:, 1536:2048], kw, 1e-6))


@pytest.mark.gpu
def test_rmsnorm_feeds_the_prologue():
    """kv_out of this operator is the kv input of the prologue: the chain equals the oracle chain."""
    from flaggems_vllm.testing import workloads

    w = workloads.make("cpu_ref", device=DEV, seed=7, num_tokens=64, num_heads=4, num_blocks=4)
    g = torch.Generator().manual_seed(8)
    qr = torch.randn(64, 1536, generator=g).to(torch.bfloat16)
    qw, kw = (1 + 0.1 * torch.randn(1536, generator=g)).to(torch.bfloat16), (1 + 0.1 * torch.randn(512, generator=g)).to(torch.bfloat16)
    _, kv_n = flaggems_vllm.fused_q_kv_rmsnorm(qr.to(DEV), w.kv, qw.to(DEV), kw.to(DEV), 1e-6)
    kv_ref = c_oracle.weighted_rmsnorm(w.kv.cpu(), kw, 1e-6)
    assert_within_one_ulp(kv_n.cpu(), kv_ref)
    kc_ref = w.k_cache.cpu().clone()
    c_oracle.prologue(w.q.cpu().clone(), kv_n.cpu(), kc_ref, w.slot_mapping.cpu(), w.position_ids.cpu(),
                      w.cos_sin_cache.cpu(), w.eps, 64)
    flaggems_vllm.fused_deepseek_v4_qnorm_rope_kv_rope_quant_insert(w.q, kv_n, w.k_cache, w.slot_mapping, w.position_ids,
                                                                  w.cos_sin_cache, w.eps, 64)
    assert torch.equal(w.k_cache.cpu(), kc_ref)


def _statement(x, weight, eps):
    """The torch statement of the operator in the upstream test (tests/test_deepseek_v4_attention_fused_q_kv_rmsnorm.py:40-44)."""
    y = x.float() * torch.rsqrt(torch.mean(x.float() * x.float(), dim=-1, keepdim=True) + eps)
    return (y * weight.float()).to(x.dtype)


@pytest.mark.gpu
@pytest.mark.parametrize("q_dtype,kv_dtype,w_dtype", [
    (torch.float16, torch.float16, torch.float16), (torch.float32, torch.float32, torch.float32),
    (torch.bfloat16, torch.bfloat16, torch.float32), (torch.float16, torch.bfloat16, torch.float32),
    (torch.float32, torch.float16, torch.bfloat16)])
@pytest.mark.parametrize("tokens,qdim,kvdim", [(1, 7, 3), (33, 1536, 512), (5, 2500, 130)])
def test_element_types_the_reference_kernel_accepts(q_dtype, kv_dtype, w_dtype, tokens, qdim, kvdim):
    """Rows and weights in float16 / float32 / bfloat16, each tensor its own (the reference kernel loads everything as
    fp32 and stores in the row's type).  Compared with the upstream test's torch statement on the same device; the
    mean's summation order is free, so the bar is one unit in the last place of the row's type (float32: 4 ulps, the
    reciprocal square root adds its own)."""
    g = torch.Generator(device="cuda:0").manual_seed(tokens * 1000 + qdim)
    qr = torch.randn(tokens, qdim, generator=g, device="cuda:0").to(q_dtype)
    kv = (torch.randn(tokens, kvdim, generator=g, device="cuda:0") * 3).to(kv_dtype)
    qw = torch.randn(qdim, generator=g, device="cuda:0").to(w_dtype)
    kw = torch.randn(kvdim, generator=g, device="cuda:0").to(w_dtype)
    q_out, kv_out = flaggems_vllm.fused_q_kv_rmsnorm(qr, kv, qw, kw, 1e-6)
    assert q_out.dtype == q_dtype and kv_out.dtype == kv_dtype and q_out.shape == qr.shape and kv_out.shape == kv.shape
    for got, want in ((q_out, _statement(qr, qw, 1e-6)), (kv_out, _statement(kv, kw, 1e-6))):
        if got.dtype == torch.float32:
            torch.testing.assert_close(got, want, rtol=5e-7, atol=0)
        else:
            ints = torch.int16
            a, b = got.view(ints).to(torch.int32), want.view(ints).to(torch.int32)
            a, b = torch.where(a < 0, -(a & 0x7FFF), a), torch.where(b < 0, -(b & 0x7FFF), b)
            d = (a - b).abs()
            assert int(d.max()) <= 1 and float((d != 0).float().mean()) < 2e-3


def test_host_checks_without_gpu():
    qr, kv = torch.zeros(4, 256, dtype=torch.bfloat16), torch.zeros(4, 128, dtype=torch.bfloat16)
    qw, kw = torch.ones(256, dtype=torch.bfloat16), torch.ones(128, dtype=torch.bfloat16)
    with pytest.raises(AssertionError, match="no CPU path"):
        flaggems_vllm.fused_q_kv_rmsnorm(qr, kv, qw, kw, 1e-6)
    with pytest.raises(AssertionError):
        flaggems_vllm.fused_q_kv_rmsnorm(qr, kv[:3], qw, kw, 1e-6)
    with pytest.raises(AssertionError):
        flaggems_vllm.fused_q_kv_rmsnorm(qr.t(), kv, qw, kw, 1e-6)
