"""`fused_inv_rope_fp8_quant`: oracle vs vectors from the upstream test's torch statement; CUDA kernel vs
both, bit for bit (bytes and scales), plus the output-layout contract of the upstream tests."""
from __future__ import annotations

import numpy as np
import pytest
import torch

import flaggems_vllm
from conftest import GOLDEN, _bf16
from flaggems_vllm.testing import workloads
from oracle import c_oracle

NAMES = sorted(p.stem for p in GOLDEN.glob("inv_rope_*.npz"))
DEV = "cuda:0"


def load(name):
    z = np.load(GOLDEN / f"{name}.npz")
    g = {"o": _bf16(z["o"]), "positions": torch.from_numpy(z["positions"].copy()), "n_groups": int(z["n_groups"]),
         "heads_per_group": int(z["heads_per_group"])}
    for k in ("fp8_0", "scale_0", "fp8_1", "scale_1"):
        g[k] = torch.from_numpy(z[k].copy())
    return g


def test_golden_files_exist():
    assert len(NAMES) >= 4


def test_pow2_scale_bit_derivation_equals_log_statement_for_every_bf16_amax():
    """The kernel takes ceil(log2(s)) of s = max(amax, eps)/448-by-reciprocal from the bits of s; the reference
    uses log2/ceil/exp2.  Equal for every non-negative finite bf16 amax."""
    amax = torch.arange(0, 0x7F80, dtype=torch.int32).to(torch.int16).view(torch.bfloat16).float()
    s = (amax.clamp(min=1e-10) * (1.0 / 448.0)).clamp(min=1e-10)
    want = torch.exp2(torch.ceil(torch.log2(s)))
    bits = s.view(torch.int32)
    code = ((bits >> 23) & 0xFF) + ((bits & 0x7FFFFF) != 0).to(torch.int32)
    got = (code << 23).view(torch.float32)
    assert torch.equal(got, want)


@pytest.mark.parametrize("form", [2, 3])
@pytest.mark.parametrize("y_ulps", [-1, 0, 1])
def test_division_shortcut_never_changes_a_byte(form, y_ulps):
    """fp32-scale mode forms x / scale from a refined reciprocal - two instructions per value (form 2, scales up to
    2^100) or three (form 3, any scale) - instead of an IEEE division.  Every reachable (scale, value) pair for bf16
    inputs and the reference's eps, for each value the device's reciprocal can take (within one ulp of the correctly
    rounded one): no e4m3 byte differs."""
    enough = 4.5e8 if form == 2 else 5.3e8  # form 2 leaves out the group maxima above 2^108
    pairs, byte_mismatches, _ = c_oracle.check_division_shortcut(1e-10, form, y_ulps)
    assert pairs > enough and byte_mismatches == 0
    # per_token_group_quant_fp8 uses the same shortcut with eps rounded to bf16 (its statement clamps a bf16 tensor)
    eps_bf16 = float(torch.tensor(1e-10).to(torch.bfloat16))
    pairs, byte_mismatches, _ = c_oracle.check_division_shortcut(eps_bf16, form, y_ulps)
    assert pairs > enough and byte_mismatches == 0


@pytest.mark.parametrize("packed", [False, True])
@pytest.mark.parametrize("name", NAMES)
def test_oracle_reproduces_upstream_reference(name, packed):
    g = load(name)
    fp8, scales = c_oracle.inv_rope_fp8_quant(g["o"], g["positions"], workloads.cos_sin_table(4096), g["n_groups"],
                                              g["heads_per_group"], packed=packed)
    assert torch.equal(fp8, g[f"fp8_{int(packed)}"])
    want = g[f"scale_{int(packed)}"]
    assert torch.equal(scales.view(torch.int32), want.view(torch.int32))


def run_kernel(o, positions, cs, n_groups, hpg, packed):
    return flaggems_vllm.fused_inv_rope_fp8_quant(o.to(DEV), positions.to(DEV), cs.to(DEV), n_groups, hpg,
                                                  tma_aligned_scales=packed)


@pytest.mark.gpu
@pytest.mark.parametrize("packed", [False, True])
@pytest.mark.parametrize("name", NAMES)
def test_kernel_reproduces_upstream_reference(name, packed):
    g = load(name)
    fp8, scale = run_kernel(g["o"], g["positions"], workloads.cos_sin_table(4096), g["n_groups"], g["heads_per_group"], packed)
    assert torch.equal(fp8.cpu().view(torch.uint8), g[f"fp8_{int(packed)}"])
    assert torch.equal(scale.cpu().contiguous().view(torch.int32), g[f"scale_{int(packed)}"].view(torch.int32))


@pytest.mark.gpu
@pytest.mark.parametrize("packed", [False, True])
@pytest.mark.parametrize("tokens,heads,groups", [(1, 64, 8), (7, 64, 8), (32, 128, 8), (128, 32, 4), (1001, 16, 1), (2, 3, 3)])
def test_kernel_matches_oracle_and_layout_contract(tokens, heads, groups, packed):
    g = torch.Generator().manual_seed(tokens * 131 + heads)
    o = torch.randn(tokens, heads, 512, generator=g).to(torch.bfloat16)
    pos = torch.randint(0, 4096, (tokens,), generator=g)
    cs = workloads.cos_sin_table(4096)
    hpg, d = heads // groups, heads // groups * 512
    fp8, scale = run_kernel(o, pos, cs, groups, hpg, packed)
    want_fp8, want_scale = c_oracle.inv_rope_fp8_quant(o, pos, cs, groups, hpg, packed=packed)
    assert torch.equal(fp8.cpu().view(torch.uint8), want_fp8)
    assert torch.equal(scale.cpu().contiguous().view(torch.int32), want_scale.view(torch.int32))
    # layout contract (upstream test_output_layout / test_per_group_contiguity)
    assert fp8.shape == (tokens, groups, d) and fp8.stride() == (d, tokens * d, 1) and fp8.dtype == torch.float8_e4m3fn
    assert scale.shape == (tokens, groups, hpg if packed else hpg * 4)
    assert scale.dtype == (torch.int32 if packed else torch.float32)
    assert scale.permute(1, 0, 2).stride(1) == 1 or tokens == 1
    assert all(fp8[:, gi, :].is_contiguous() for gi in range(groups))
    # the token padding of the scale storage (multiple of 4) is zeroed
    padded = (tokens + 3) // 4 * 4
    k = scale.shape[2]
    storage = torch.as_strided(scale, (groups, k, padded), (k * padded, padded, 1))
    assert int((storage[:, :, tokens:].view(torch.int32) != 0).sum()) == 0


@pytest.mark.gpu
def test_strided_input_and_read_only():
    """o as a view with a larger token stride; o itself is not modified."""
    g = torch.Generator().manual_seed(9)
    big = torch.randn(10, 20, 512, generator=g).to(torch.bfloat16)
    pos = torch.randint(0, 4096, (10,), generator=g)
    cs = workloads.cos_sin_table(4096)
    d_big = big.to(DEV)
    view = d_big[:, 2:18, :]
    fp8, scale = flaggems_vllm.fused_inv_rope_fp8_quant(view, pos.to(DEV), cs.to(DEV), 4, 4)
    assert torch.equal(d_big.cpu(), big)
    want_fp8, want_scale = c_oracle.inv_rope_fp8_quant(big[:, 2:18, :], pos, cs, 4, 4)
    assert torch.equal(fp8.cpu().view(torch.uint8), want_fp8) and torch.equal(scale.cpu().contiguous(), want_scale)


@pytest.mark.gpu
def test_inverse_of_the_prologue_rotation():
    """Rotating with the prologue and un-rotating with this operator returns the un-rotated tail up to bf16
    rounding: de-quantised tail of inv(rope(x)) is close to the RMS-normalised x tail."""
    w = workloads.make("cpu_ref", device=DEV, seed=11, num_tokens=32, num_heads=8, num_blocks=2)
    q0 = w.q.clone()
    flaggems_vllm.fused_deepseek_v4_qnorm_rope_kv_rope_quant_insert(*w.args())
    fp8, scale = flaggems_vllm.fused_inv_rope_fp8_quant(w.q, w.position_ids, w.cos_sin_cache, 1, 8)
    deq = fp8.float().view(32, 8, 4, 128) * scale.view(32, 8, 4, 1)
    normed = q0.float() * torch.rsqrt(q0.float().pow(2).mean(-1, keepdim=True) + 1e-6)
    err = (deq.view(32, 8, 512)[..., 448:] - normed[..., 448:]).abs()
    assert float(err.max()) < 0.3 and float(err.mean()) < 0.03  # e4m3 step at |x| ~ 4 is 0.25


@pytest.mark.gpu
@pytest.mark.parametrize("eps", [1e-10, 1e-4])
def test_fp32_scale_mode_with_and_without_the_division_shortcut(eps):
    """eps = 1e-10 takes the shortcut, any other eps the IEEE division; both must equal the oracle, on values of
    widely different magnitude (tiny groups hit the eps clamp)."""
    g = torch.Generator().manual_seed(77)
    o = (torch.randn(257, 16, 512, generator=g) * torch.logspace(-8, 4, 257)[:, None, None]).to(torch.bfloat16)
    pos = torch.randint(0, 4096, (257,), generator=g)
    cs = workloads.cos_sin_table(4096)
    fp8, scale = flaggems_vllm.fused_inv_rope_fp8_quant(o.to(DEV), pos.to(DEV), cs.to(DEV), 2, 8, eps=eps)
    want_fp8, want_scale = c_oracle.inv_rope_fp8_quant(o, pos, cs, 2, 8, eps=eps)
    assert torch.equal(fp8.cpu().view(torch.uint8), want_fp8)
    assert torch.equal(scale.cpu().contiguous().view(torch.int32), want_scale.view(torch.int32))


def test_host_checks_without_gpu():
    o = torch.zeros(4, 8, 512, dtype=torch.bfloat16)
    pos = torch.zeros(4, dtype=torch.int64)
    cs = torch.zeros(16, 64)
    with pytest.raises(AssertionError, match="no CPU path"):
        flaggems_vllm.fused_inv_rope_fp8_quant(o, pos, cs, 2, 4)
    with pytest.raises(AssertionError):
        flaggems_vllm.fused_inv_rope_fp8_quant(o, pos, cs, 3, 4)
    with pytest.raises(AssertionError):
        flaggems_vllm.fused_inv_rope_fp8_quant(o, pos[:3], cs, 2, 4)
    with pytest.raises(AssertionError):
        flaggems_vllm.fused_inv_rope_fp8_quant(o, pos, cs, 2, 4, nope_dim=384, rope_dim=128)
    assert flaggems_vllm.ops_inv_rope_fp8_quant is flaggems_vllm.fused_inv_rope_fp8_quant
