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


@pytest.mark.gpu
@pytest.mark.parametrize("form", [2, 3])
@pytest.mark.parametrize("eps_rounded_to_bf16", [False, True])
def test_division_shortcut_on_the_device_itself(form, eps_rounded_to_bf16):
    """The same enumeration as the CPU proof above, run by the GPU with its own approximate reciprocal: every bf16 group
    maximum against every bf16 value below it - no e4m3 byte differs from the IEEE quotient's, and the refined reciprocal
    is within one unit in the last place of the correctly rounded one for every scale (the premise of the CPU proof)."""
    from flaggems_vllm.testing import hbm_probe

    eps = float(torch.tensor(1e-10).to(torch.bfloat16)) if eps_rounded_to_bf16 else 1e-10
    counts = torch.zeros(3, dtype=torch.int64, device=DEV)
    hbm_probe.division_probe(eps, form, counts.data_ptr(), torch.cuda.current_stream().cuda_stream)
    pairs, byte_mismatches, reciprocals_off = counts.cpu().tolist()
    assert pairs > (4.5e8 if form == 2 else 5.3e8)
    assert byte_mismatches == 0 and reciprocals_off == 0


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


# geometries other than the DeepSeek-V4 one that pass the reference wrapper's assertions: (nope, rope, group)
GEOMETRIES = [(192, 64, 128), (64, 64, 128), (192, 64, 64), (96, 32, 64), (224, 32, 64), (120, 8, 32), (0, 128, 128), (384, 128, 256)]


def _cos_sin_any(max_pos: int, rope_dim: int) -> torch.Tensor:
    half = rope_dim // 2
    freqs = 1.0 / (10000.0 ** (torch.arange(0, half, dtype=torch.float32) * 2 / rope_dim))
    angles = torch.arange(max_pos, dtype=torch.float32)[:, None] * freqs[None, :]
    return torch.cat([angles.cos(), angles.sin()], dim=-1).contiguous()


def _statement_any(o, pos, cs, groups, hpg, nope, rope, group, packed):
    """The upstream test's torch statement (tests/test_fused_inv_rope_fp8_quant.py:132-198 upstream) written for any
    rotary width: its `native_fused_inv_rope_fp8_quant` fixes the width at 64, its `_reference_inv_rope` does not."""
    half = rope // 2
    sel = cs.index_select(0, pos)
    cos = sel[:, :half].repeat_interleave(2, dim=-1).unsqueeze(1)
    sin = -sel[:, half:].repeat_interleave(2, dim=-1).unsqueeze(1)
    tail = o[..., nope:].float()
    swapped = torch.stack((-tail[..., 1::2], tail[..., ::2]), dim=-1).flatten(-2)
    rot = torch.cat((o[..., :nope], (tail * cos + swapped * sin).to(o.dtype)), dim=-1)
    tokens, _, head_dim = rot.shape
    blocks = rot.view(tokens, groups, hpg * head_dim // group, group).float()
    scales = blocks.abs().amax(dim=-1).clamp(min=1e-10) * (1.0 / 448.0)
    if packed:
        scales = torch.exp2(torch.ceil(torch.log2(scales.clamp(min=1e-10))))
    fp8 = (blocks / scales.unsqueeze(-1)).clamp(-448.0, 448.0).to(torch.float8_e4m3fn).reshape(tokens, groups, hpg * head_dim)
    if packed:
        codes = (scales.view(torch.int32) >> 23) & 0xFF
        codes = codes.reshape(tokens, groups, hpg, head_dim // group)
        scales = sum(codes[..., j] << (8 * j) for j in range(head_dim // group)).to(torch.int32)
    return fp8.view(torch.uint8), scales


@pytest.mark.parametrize("nope,rope,group", GEOMETRIES)
@pytest.mark.parametrize("packed", [False, True])
def test_oracle_follows_the_statement_for_other_geometries(nope, rope, group, packed):
    if packed and (nope + rope) // group != 4:
        pytest.skip("packed scales are defined for four groups per head only")
    g = torch.Generator().manual_seed(nope + rope + group)
    tokens, groups, hpg = 9, 2, 3
    o = (torch.randn(tokens, groups * hpg, nope + rope, generator=g) * torch.logspace(-3, 2, tokens)[:, None, None]).to(torch.bfloat16)
    pos = torch.randint(0, 512, (tokens,), generator=g)
    cs = _cos_sin_any(512, rope)
    want_fp8, want_scale = _statement_any(o, pos, cs, groups, hpg, nope, rope, group, packed)
    fp8, scale = c_oracle.inv_rope_fp8_quant(o, pos, cs, groups, hpg, packed=packed, nope_dim=nope, rope_dim=rope, quant_group_size=group)
    assert torch.equal(fp8, want_fp8)
    assert torch.equal(scale.view(torch.int32), want_scale.contiguous().view(torch.int32))


@pytest.mark.gpu
@pytest.mark.parametrize("nope,rope,group", GEOMETRIES)
@pytest.mark.parametrize("packed", [False, True])
@pytest.mark.parametrize("tokens,heads,groups", [(1, 4, 2), (37, 12, 3), (130, 8, 8)])
def test_other_geometries_match_the_oracle(nope, rope, group, packed, tokens, heads, groups):
    """Every geometry the reference wrapper accepts runs (on a general kernel) and matches the oracle bit for bit,
    fp8 bytes, scales, layout and the zeroed token padding of the scale storage."""
    chunks = (nope + rope) // group
    if packed and chunks != 4:
        pytest.skip("packed scales are defined for four groups per head only")
    g = torch.Generator().manual_seed(tokens * 7 + nope + group)
    head_dim, hpg = nope + rope, heads // groups
    o = (torch.randn(tokens, heads, head_dim, generator=g) * torch.logspace(-2, 2, tokens)[:, None, None]).to(torch.bfloat16)
    pos = torch.randint(0, 512, (tokens,), generator=g)
    cs = _cos_sin_any(512, rope)
    fp8, scale = flaggems_vllm.fused_inv_rope_fp8_quant(o.to(DEV), pos.to(DEV), cs.to(DEV), groups, hpg, nope_dim=nope, rope_dim=rope,
                                                        quant_group_size=group, tma_aligned_scales=packed)
    want_fp8, want_scale = c_oracle.inv_rope_fp8_quant(o, pos, cs, groups, hpg, packed=packed, nope_dim=nope, rope_dim=rope,
                                                       quant_group_size=group)
    assert torch.equal(fp8.cpu().view(torch.uint8), want_fp8)
    assert torch.equal(scale.cpu().contiguous().view(torch.int32), want_scale.view(torch.int32))
    d = hpg * head_dim
    assert fp8.shape == (tokens, groups, d) and fp8.stride() == (d, tokens * d, 1)
    assert scale.shape == (tokens, groups, hpg if packed else hpg * chunks)
    padded, k = (tokens + 3) // 4 * 4, scale.shape[2]
    storage = torch.as_strided(scale, (groups, k, padded), (k * padded, padded, 1))
    assert int((storage[:, :, tokens:].view(torch.int32) != 0).sum()) == 0


@pytest.mark.gpu
def test_unaligned_rows_of_the_deepseek_geometry_take_the_general_kernel():
    """448 + 64 / 128 with rows that do not start on 16 bytes (a view one element into its storage)."""
    g = torch.Generator().manual_seed(5)
    flat = torch.randn(6 * 4 * 512 + 1, generator=g).to(torch.bfloat16)
    pos = torch.randint(0, 4096, (6,), generator=g)
    cs = workloads.cos_sin_table(4096)
    view = flat.to(DEV)[1:].view(6, 4, 512)
    assert view.data_ptr() % 16 != 0
    fp8, scale = flaggems_vllm.fused_inv_rope_fp8_quant(view, pos.to(DEV), cs.to(DEV), 2, 2)
    want_fp8, want_scale = c_oracle.inv_rope_fp8_quant(flat[1:].view(6, 4, 512), pos, cs, 2, 2)
    assert torch.equal(fp8.cpu().view(torch.uint8), want_fp8) and torch.equal(scale.cpu().contiguous(), want_scale)


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
