"""The CPU oracles against the golden vectors made by the upstream torch reference, and the
scalar conversions of the C oracle against torch itself.  No GPU."""
from __future__ import annotations

import hashlib

import numpy as np
import torch

from conftest import GOLDEN, _bf16
from flaggems_vllm.testing import compare, workloads
from oracle import c_oracle, torch_path


def _run(fn, g):
    q, kc = g["q"].clone(), g["k_cache"].clone()
    kv_before = g["kv"].clone()
    fn(q, g["kv"], kc, g["slot_mapping"], g["position_ids"], g["cos_sin_cache"], g["eps"], g["block_size"])
    assert torch.equal(g["kv"], kv_before), "kv is read-only"
    return q, kc


def test_torch_path_reproduces_upstream_bit_for_bit(golden_case):
    _, g = golden_case
    q, kc = _run(torch_path.prologue, g)
    assert torch.equal(q.view(torch.int16), g["q_out"].view(torch.int16))
    assert torch.equal(kc, g["k_cache_out"])


def test_c_oracle_matches_upstream(golden_case):
    """Cache bytes identical; q within 1 bf16 ulp (the fp32 summation order of torch's mean is
    not specified, the C oracle uses the correctly rounded sum)."""
    _, g = golden_case
    q, kc = _run(c_oracle.prologue, g)
    assert torch.equal(kc, g["k_cache_out"])
    st = compare.assert_q_close(q, g["q_out"], max_ulp=1, max_fraction=1e-3)
    assert st["max_ulp"] <= 1


def _sha(t):
    return hashlib.sha256(t.contiguous().view(torch.uint8).numpy().tobytes()).hexdigest()


def test_cpu_ref_config_against_upstream_digests():
    """The benchmark configuration "CPU torch reference path, seed 0": 256 tokens x 8 heads."""
    z = np.load(GOLDEN / "cpu_ref.npz")
    w = workloads.make("cpu_ref", device="cpu", seed=0)
    got = [_sha(t) for t in (w.q, w.kv, w.k_cache, w.slot_mapping, w.position_ids)]
    assert got == list(z["input_sha"]), "seeded inputs differ from the ones the golden vectors were made from"

    q, kc = w.q.clone(), w.k_cache.clone()
    torch_path.prologue(q, w.kv, kc, w.slot_mapping, w.position_ids, w.cos_sin_cache, w.eps, w.cache_block_size)
    assert _sha(q) == str(z["q_out_sha"]) and _sha(kc) == str(z["k_cache_out_sha"])

    q2, kc2 = w.q.clone(), w.k_cache.clone()
    c_oracle.prologue(q2, w.kv, kc2, w.slot_mapping, w.position_ids, w.cos_sin_cache, w.eps, w.cache_block_size)
    assert _sha(kc2) == str(z["k_cache_out_sha"])
    compare.assert_q_close(q2, q, max_ulp=1, max_fraction=1e-3)
    assert torch.equal(q[:48].view(torch.int16), _bf16(z["q_out_head"]).view(torch.int16))
    d, s = compare.gather_rows(kc2, w.slot_mapping, 64)
    assert torch.equal(d, torch.from_numpy(z["rows_data"])) and torch.equal(s, torch.from_numpy(z["rows_scales"]))
    compare.assert_untouched(kc2, w.k_cache, w.slot_mapping, 64)


def test_e4m3_conversion_matches_torch():
    """Every bf16-representable value in the finite e4m3 range, plus random floats (ties, subnormals)."""
    bits = torch.arange(0, 1 << 16, dtype=torch.int32).to(torch.int16)
    x = bits.view(torch.bfloat16).float()
    x = x[torch.isfinite(x) & (x.abs() <= 448.0)]
    g = torch.Generator().manual_seed(0)
    r = torch.cat([
        x,
        (torch.rand(1 << 18, generator=g) - 0.5) * 896.0,
        (torch.rand(1 << 16, generator=g) - 0.5) * 0.05,
        torch.arange(-448, 449, dtype=torch.float32) / 1.0,
        torch.arange(0, 64, dtype=torch.float32) * 2.0 ** -10,  # every subnormal tie
        torch.tensor([17.0, 19.0, 2.0 ** -10, 0.75 * 2.0 ** -9, 464.0, -464.0, 0.0, -0.0]),
    ])
    r = r.clamp(-448.0, 448.0)
    want = r.to(torch.float8_e4m3fn).view(torch.uint8)
    assert torch.equal(c_oracle.e4m3_from_f32(r), want)
    back = want.view(torch.float8_e4m3fn).float()
    assert torch.equal(c_oracle.f32_from_e4m3(want), back)


def test_bf16_rounding_matches_torch():
    g = torch.Generator().manual_seed(1)
    x = torch.cat([torch.randn(1 << 18, generator=g) * 10.0, torch.tensor([1.00390625, 1.01171875, 0.0, -0.0, 3.3895e38])])
    assert torch.equal(c_oracle.bf16_from_f32(x).view(torch.int16), x.to(torch.bfloat16).view(torch.int16))


def test_ue8m0_bit_derivation_equals_log_statement_for_every_bf16_and_fp16():
    """The CUDA kernels derive the scale byte from the exponent and mantissa of max(amax, 1e-4) (448 = 1.75 * 2^8);
    the reference states it as ceil(log2(. / 448)).  They agree for all non-negative finite bf16 and fp16
    magnitudes, and both agree with torch's log2/ceil."""
    bf16 = torch.arange(0, 0x7F80, dtype=torch.int32).to(torch.int16).view(torch.bfloat16).float()
    fp16 = torch.arange(0, 0x7C00, dtype=torch.int32).to(torch.int16).view(torch.float16).float()
    for amax in (bf16, fp16):
        by_log, by_bits = c_oracle.ue8m0_codes(amax)
        assert torch.equal(by_log, by_bits)
        want = (torch.ceil(torch.log2(amax.clamp(min=1e-4) / 448.0)) + 127.0).clamp(0, 255).to(torch.uint8)
        assert torch.equal(by_log, want)
        assert int(by_log.min()) >= 105 and int(by_log.max()) <= 247  # never reaches the clamps


def test_gather_dequant_oracle_inverts_the_insert(golden_case):
    """Reader oracle on the upstream-written cache: bf16 RoPE part identical to the stored bytes,
    de-quantised part within half a quantisation step of the original kv."""
    name, g = golden_case
    slots = compare.valid_slots(g["slot_mapping"])
    if slots.numel() == 0:
        return
    bs = g["block_size"]
    rows = c_oracle.gather_dequant(g["k_cache_out"], slots, bs)
    d, s = compare.gather_rows(g["k_cache_out"], slots, bs)
    assert torch.equal(rows[:, 448:].contiguous().view(torch.uint8), d[:, 448:].contiguous())
    scale = torch.exp2(s[:, :7].float() - 127.0).repeat_interleave(64, dim=1)
    want = (d[:, :448].contiguous().view(torch.float8_e4m3fn).float() * scale).to(torch.bfloat16)
    assert torch.equal(rows[:, :448].view(torch.int16), want.view(torch.int16))
    n_ins = g["slot_mapping"].shape[0]
    kv_valid = g["kv"][:n_ins][g["slot_mapping"] >= 0][:, :448].float()
    # e4m3 keeps 3 mantissa bits: relative error <= 2^-4, plus half a subnormal step (2^-10) of the scale
    err = (rows[:, :448].float() - kv_valid).abs()
    assert bool((err <= kv_valid.abs() * 2.0 ** -4 + scale * 2.0 ** -10 + 1e-30).all())


def test_oracles_reproduce_the_upstream_flash_mla_cache_builder():
    """An independent upstream statement of the cache format and quantiser (the FlashMLA test's cache builder): with an
    identity rotation (cos 1, sin 0) the oracles must produce its cache byte for byte from the keys it drew."""
    z = np.load(GOLDEN / "flash_mla_builder_cache.npz")
    kv = torch.from_numpy(z["kv"].view(np.int16).copy()).view(torch.bfloat16)
    want, bs, n = torch.from_numpy(z["cache"].copy()), int(z["block_size"]), kv.shape[0]
    table = torch.cat([torch.ones(2, 32), torch.zeros(2, 32)], dim=1).contiguous()
    for run in (c_oracle.prologue, torch_path.prologue):
        cache = torch.zeros_like(want)
        run(torch.ones(n, 1, 512, dtype=torch.bfloat16), kv, cache, torch.arange(n), torch.zeros(n, dtype=torch.int64), table, 1e-6, bs)
        assert torch.equal(cache, want)
