"""`fused_indexer_q_rope_quant`: oracle vs vectors from the upstream test's torch statements (FP8 and MXFP4);
CUDA kernel vs both, bit for bit as the upstream test demands (values, scales, weights rtol=0 atol=0)."""
from __future__ import annotations

import numpy as np
import pytest
import torch

import flaggems_vllm
from conftest import GOLDEN, _bf16
from oracle import c_oracle

NAMES = sorted(p.stem for p in GOLDEN.glob("indexer_q_*.npz"))
DEV = "cuda:0"
SM, HS = 128 ** -0.5, 8 ** -0.5


def table(max_pos, rot_dim, dtype):
    half = rot_dim // 2
    inv = 1.0 / (10000.0 ** (torch.arange(0, half, dtype=torch.float32) / half))
    ang = torch.outer(torch.arange(max_pos, dtype=torch.float32), inv)
    return torch.cat((ang.cos(), ang.sin()), dim=-1).to(dtype)


def load(name):
    z = np.load(GOLDEN / f"{name}.npz")
    g = {"q": _bf16(z["q"]), "positions": torch.from_numpy(z["positions"].copy()), "weights": _bf16(z["weights"]),
         "cs": table(4096, 64, torch.bfloat16 if int(z["table_bf16"]) else torch.float32)}
    for k in ("fp8", "w_fp8", "fp4", "fp4_scales", "w_fp4"):
        g[k] = torch.from_numpy(z[k].copy())
    return g


def test_golden_files_exist():
    assert len(NAMES) == 6


def test_mxfp4_scale_bit_derivation_equals_log_statement_for_every_bf16_amax():
    amax = torch.arange(0, 0x7F80, dtype=torch.int32).to(torch.int16).view(torch.bfloat16).float()
    r = amax.clamp(min=6 * 2.0 ** -126) / 6.0
    want = (r.log2().ceil().clamp(-127.0, 127.0) + 127.0).to(torch.int32)
    # the kernel's division-free form: 6 = 1.5 * 4 -> exponent of the clamped maximum minus 2, plus 1 if mantissa > 1.5
    bits = amax.clamp(min=6 * 2.0 ** -126).view(torch.int32)
    got = ((bits >> 23) - 2 + ((bits & 0x7FFFFF) > 0x400000).to(torch.int32)).clamp(max=254)
    assert torch.equal(got, want)


@pytest.mark.parametrize("name", NAMES)
def test_oracle_reproduces_upstream_reference(name):
    g = load(name)
    out, _, w = c_oracle.indexer_q_rope_quant(g["positions"], g["q"], g["cs"], g["weights"], SM, HS, use_fp4=False)
    assert torch.equal(out, g["fp8"]) and torch.equal(w, g["w_fp8"])
    out, scales, w = c_oracle.indexer_q_rope_quant(g["positions"], g["q"], g["cs"], g["weights"], SM, HS, use_fp4=True)
    assert torch.equal(out, g["fp4"]) and torch.equal(w, g["w_fp4"])
    assert torch.equal(scales.view(torch.int32).squeeze(-1), g["fp4_scales"])


@pytest.mark.gpu
@pytest.mark.parametrize("name", NAMES)
def test_kernel_reproduces_upstream_reference(name):
    g = load(name)
    args = (g["positions"].to(DEV), g["q"].to(DEV), g["cs"].to(DEV), g["weights"].to(DEV), SM, HS)
    q8, w8 = flaggems_vllm.fused_indexer_q_rope_quant(*args)
    assert q8.dtype == torch.float8_e4m3fn and w8.dtype == torch.float32
    assert torch.equal(q8.cpu().view(torch.uint8), g["fp8"]) and torch.equal(w8.cpu(), g["w_fp8"])
    (q4, s4), w4 = flaggems_vllm.fused_indexer_q_rope_quant(*args, use_fp4=True)
    assert q4.dtype == torch.uint8 and s4.dtype == torch.int32 and s4.shape == g["fp4_scales"].shape
    assert torch.equal(q4.cpu(), g["fp4"]) and torch.equal(s4.cpu(), g["fp4_scales"]) and torch.equal(w4.cpu(), g["w_fp4"])


@pytest.mark.gpu
@pytest.mark.parametrize("use_fp4", [False, True])
@pytest.mark.parametrize("tokens,heads,head_dim,rot_dim,wdtype,tdtype", [
    (1, 64, 128, 64, torch.bfloat16, torch.float32), (1000, 64, 128, 64, torch.bfloat16, torch.float32),
    (33, 8, 128, 64, torch.float32, torch.bfloat16), (17, 4, 64, 32, torch.float16, torch.float32),
    (19, 3, 256, 64, torch.bfloat16, torch.float32), (8, 8, 128, 128, torch.bfloat16, torch.float32),
    (8, 8, 128, 0, torch.bfloat16, torch.float32),
    # 8192 tokens and more take the warp-per-token kernel (even and odd head counts, both table dtypes)
    (8195, 8, 128, 64, torch.bfloat16, torch.float32), (8192, 7, 128, 64, torch.float32, torch.bfloat16),
    (9000, 1, 128, 64, torch.float16, torch.float32),
])
def test_kernel_matches_oracle(tokens, heads, head_dim, rot_dim, wdtype, tdtype, use_fp4):
    g = torch.Generator().manual_seed(tokens * 7 + head_dim + rot_dim)
    q = (torch.randn(tokens, heads, head_dim, generator=g) * torch.logspace(-3, 3, min(tokens, 64)).repeat((tokens + 63) // 64)[:tokens, None, None]).to(torch.bfloat16)
    pos = torch.randint(0, 2048, (tokens,), generator=g, dtype=torch.int64)
    cs = table(2048, rot_dim, tdtype) if rot_dim else torch.zeros(2048, 0, dtype=tdtype)
    w = torch.randn(tokens, heads, generator=g).to(wdtype)
    want_q, want_s, want_w = c_oracle.indexer_q_rope_quant(pos, q, cs, w, 0.1, 0.5, use_fp4=use_fp4)
    res, w_out = flaggems_vllm.fused_indexer_q_rope_quant(pos.to(DEV), q.to(DEV), cs.to(DEV), w.to(DEV), 0.1, 0.5, use_fp4=use_fp4)
    assert torch.equal(w_out.cpu(), want_w)
    if use_fp4:
        assert torch.equal(res[0].cpu(), want_q)
        assert torch.equal(res[1].cpu().contiguous().view(torch.uint8).view(tokens, heads, -1), want_s)
    else:
        assert torch.equal(res.cpu().view(torch.uint8), want_q)


@pytest.mark.gpu
def test_strided_index_q():
    g = torch.Generator().manual_seed(3)
    big = torch.randn(12, 10, 128, generator=g).to(torch.bfloat16)
    pos = torch.randint(0, 2048, (12,), generator=g, dtype=torch.int64)
    cs, w = table(2048, 64, torch.float32), torch.randn(12, 8, generator=g).to(torch.bfloat16)
    want_q, _, want_w = c_oracle.indexer_q_rope_quant(pos, big[:, 1:9], cs, w, SM, HS)
    q8, w8 = flaggems_vllm.fused_indexer_q_rope_quant(pos.to(DEV), big.to(DEV)[:, 1:9], cs.to(DEV), w.to(DEV), SM, HS)
    assert torch.equal(q8.cpu().contiguous().view(torch.uint8), want_q) and torch.equal(w8.cpu(), want_w)


def test_host_checks_without_gpu():
    pos, q = torch.zeros(4, dtype=torch.int64), torch.zeros(4, 8, 128, dtype=torch.bfloat16)
    cs, w = torch.zeros(16, 64), torch.zeros(4, 8, dtype=torch.bfloat16)
    with pytest.raises(AssertionError, match="no CPU path"):
        flaggems_vllm.fused_indexer_q_rope_quant(pos, q, cs, w, 1.0, 1.0)
    with pytest.raises(RuntimeError, match="requires CUDA"):
        flaggems_vllm.fused_indexer_q_rope_quant(pos, q, cs, w, 1.0, 1.0, use_fp4=True)
    with pytest.raises(AssertionError):
        flaggems_vllm.fused_indexer_q_rope_quant(pos, q[0], cs, w, 1.0, 1.0)
