"""Parity comparators for the prologue operator (pure torch, any device).

They state the acceptance bars this project holds itself to:
  * query rows: every bf16 within 1 unit in the last place of the reference.  For the 64
    rotated values the unit is taken at the magnitude of the (even, odd) pair they come from:
    `e*c - o*s` can cancel, and a 1-ulp fp32 difference in 1/rms (torch's own summation order is
    unspecified) then shows up as several ulps OF THE SMALL RESULT while still being far below
    one ulp of its operands.  Such elements are counted and reported as `tail_cancellations`;
  * cached e4m3 bytes: at least 99.9 % identical, the rest adjacent codes (1 e4m3
    ulp, hence within 1 ulp after multiplying by the shared power-of-two scale);
  * UE8M0 scale bytes identical (the decoded power of two then has zero error) and
    the pad byte zero;
  * cached bf16 RoPE values within 1 ulp;
  * every byte of the cache that no valid slot addresses is bit-identical to what
    it was before the call.
The upstream tests use looser bars (rtol=atol=1e-2 on bf16, bytes exact;
tests/test_fused_deepseek_v4_qnorm_rope_kv_rope_quant_insert.py:246-289).
"""
from __future__ import annotations

import torch

TOKEN_DATA_BYTES, SCALE_BYTES, NOPE_DIM = 576, 8, 448


def _ordinal16(bits: torch.Tensor) -> torch.Tensor:
    """Sign-magnitude 16-bit patterns -> integers whose order is the numeric order."""
    b = bits.view(torch.int16).to(torch.int32) & 0xFFFF
    mag = b & 0x7FFF
    return torch.where(b >= 0x8000, -mag, mag)


def bf16_ulp_distance(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """|ordinal(a) - ordinal(b)| for bf16 tensors (+0 and -0 coincide)."""
    assert a.dtype == torch.bfloat16 and b.dtype == torch.bfloat16 and a.shape == b.shape
    return (_ordinal16(a) - _ordinal16(b)).abs()


def e4m3_code_distance(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """|ordinal(a) - ordinal(b)| for e4m3 bit patterns held in uint8 tensors."""
    ai, bi = a.to(torch.int32), b.to(torch.int32)
    oa = torch.where(ai >= 128, -(ai & 127), ai)
    ob = torch.where(bi >= 128, -(bi & 127), bi)
    return (oa - ob).abs()


def _pair_ulp(ref_tail: torch.Tensor) -> torch.Tensor:
    """bf16 ulp at the magnitude of each (even, odd) pair of a [..., 64] rotary tail."""
    pairs = ref_tail.float().unflatten(-1, (32, 2)).abs().amax(dim=-1, keepdim=True)
    _, e = torch.frexp(pairs)  # pairs = f * 2^e, f in [0.5, 1)
    return torch.ldexp(torch.ones_like(pairs), e - 8).expand(*pairs.shape[:-1], 2).flatten(-2)


def q_stats(q: torch.Tensor, q_ref: torch.Tensor, chunk_tokens: int = 2048) -> dict:
    """ulp statistics between two q tensors [N, H, 512], token-chunked.
    max_ulp: worst distance over the 448 un-rotated values and over the rotated values that did
    not cancel; tail_cancellations: rotated values more than 1 own-ulp apart yet within one ulp
    of their pair's magnitude; tail_violations: rotated values outside even that."""
    worst, differ, total, cancel, violate = 0, 0, 0, 0, 0
    has_nan = False
    for s in range(0, q.shape[0], chunk_tokens):
        a, b = q[s : s + chunk_tokens], q_ref[s : s + chunk_tokens]
        if a.numel() == 0:
            continue
        d = bf16_ulp_distance(a, b)
        differ += int((d != 0).sum().item())
        total += d.numel()
        has_nan = has_nan or bool(torch.isnan(a.float()).any().item())
        worst = max(worst, int(d[..., :NOPE_DIM].max().item()))
        tail_d = d[..., NOPE_DIM:]
        far = tail_d > 1
        if bool(far.any().item()):
            within = (a[..., NOPE_DIM:].float() - b[..., NOPE_DIM:].float()).abs() <= _pair_ulp(b[..., NOPE_DIM:])
            cancel += int((far & within).sum().item())
            violate += int((far & ~within).sum().item())
            tail_d = torch.where(far & within, torch.ones_like(tail_d), tail_d)
        worst = max(worst, int(tail_d.max().item()))
    return {"max_ulp": worst, "mismatch_fraction": differ / max(total, 1), "elements": total, "nan": has_nan,
            "tail_cancellations": cancel, "tail_violations": violate}


def assert_q_close(q, q_ref, max_ulp: int = 1, max_fraction: float = 1e-3) -> dict:
    s = q_stats(q, q_ref)
    assert not s["nan"], "NaN in q"
    assert s["tail_violations"] == 0, f"{s['tail_violations']} rotated values off by more than a pair-magnitude ulp"
    assert s["max_ulp"] <= max_ulp, f"q differs by {s['max_ulp']} bf16 ulp (allowed {max_ulp})"
    assert s["mismatch_fraction"] <= max_fraction, f"q mismatch fraction {s['mismatch_fraction']:.3e}"
    return s


def cache_views(k_cache: torch.Tensor, block_size: int):
    """(data [blocks, bs, 576], scales [blocks, bs, 8]) byte views honouring the block stride."""
    assert k_cache.dim() == 2 and k_cache.dtype == torch.uint8 and k_cache.stride(1) == 1
    nb, stride = k_cache.shape[0], k_cache.stride(0)
    assert k_cache.shape[1] >= block_size * (TOKEN_DATA_BYTES + SCALE_BYTES)
    off = k_cache.storage_offset()
    data = k_cache.as_strided((nb, block_size, TOKEN_DATA_BYTES), (stride, TOKEN_DATA_BYTES, 1), off)
    scales = k_cache.as_strided((nb, block_size, SCALE_BYTES), (stride, SCALE_BYTES, 1),
                                off + block_size * TOKEN_DATA_BYTES)
    return data, scales


def valid_slots(slot_mapping: torch.Tensor) -> torch.Tensor:
    return slot_mapping[slot_mapping >= 0]


def gather_rows(k_cache: torch.Tensor, slots: torch.Tensor, block_size: int):
    """(data rows [n,576], scale rows [n,8]) stored at `slots` (all >= 0)."""
    data, scales = cache_views(k_cache, block_size)
    blk, pos = slots // block_size, slots % block_size
    return data[blk, pos], scales[blk, pos]


def assert_untouched(k_cache, k_cache_before, slot_mapping, block_size: int) -> None:
    """Every byte outside the rows addressed by valid slots equals its old value."""
    slots = valid_slots(slot_mapping)
    patched = k_cache_before.clone()
    if slots.numel():
        pd, ps = cache_views(patched, block_size)
        ad, asc = cache_views(k_cache, block_size)
        blk, pos = slots // block_size, slots % block_size
        pd[blk, pos] = ad[blk, pos]
        ps[blk, pos] = asc[blk, pos]
    assert torch.equal(patched, k_cache), "a cache byte outside the addressed slots changed"


def cache_stats(k_cache, k_cache_ref, slot_mapping, block_size: int) -> dict:
    """Compare the rows at the valid slots of two caches."""
    slots = valid_slots(slot_mapping)
    if slots.numel() == 0:
        return {"rows": 0, "fp8_identical_fraction": 1.0, "fp8_max_code_distance": 0, "scale_bytes_equal": True,
                "pad_zero": True, "rope_max_ulp": 0, "rope_identical": True, "rope_cancellations": 0}
    d, s = gather_rows(k_cache, slots, block_size)
    dr, sr = gather_rows(k_cache_ref, slots, block_size)
    fp8, fp8r = d[:, :NOPE_DIM], dr[:, :NOPE_DIM]
    same = fp8 == fp8r
    dist = e4m3_code_distance(fp8, fp8r)
    rope = d[:, NOPE_DIM:].contiguous().view(torch.bfloat16)
    roper = dr[:, NOPE_DIM:].contiguous().view(torch.bfloat16)
    rope_d = bf16_ulp_distance(rope, roper)
    far = rope_d > 1
    cancellations = 0
    if bool(far.any().item()):  # same rule as for q: a cancelled rotation is judged at its pair's magnitude
        within = (rope.float() - roper.float()).abs() <= _pair_ulp(roper)
        cancellations = int((far & within).sum().item())
        rope_d = torch.where(far & within, torch.ones_like(rope_d), rope_d)
    return {
        "rows": int(slots.numel()),
        "fp8_identical_fraction": float(same.float().mean().item()),
        "fp8_max_code_distance": int(dist.max().item()),
        "scale_bytes_equal": bool(torch.equal(s[:, :7], sr[:, :7])),
        "pad_zero": bool((s[:, 7] == 0).all().item()),
        "rope_max_ulp": int(rope_d.max().item()),
        "rope_identical": bool(torch.equal(rope.view(torch.int16), roper.view(torch.int16))),
        "rope_cancellations": cancellations,
    }


def assert_cache_close(k_cache, k_cache_ref, slot_mapping, block_size: int, exact: bool = True) -> dict:
    """The cache bars above; `exact` additionally demands byte-identical rows (what the
    kernel is designed to deliver, since the KV path has no order-dependent arithmetic)."""
    st = cache_stats(k_cache, k_cache_ref, slot_mapping, block_size)
    assert st["scale_bytes_equal"], "UE8M0 scale bytes differ"
    assert st["pad_zero"], "scale pad byte is not zero"
    assert st["fp8_identical_fraction"] >= 0.999, f"only {st['fp8_identical_fraction']:.6f} of e4m3 bytes identical"
    assert st["fp8_max_code_distance"] <= 1, "an e4m3 byte is more than 1 ulp off"
    assert st["rope_max_ulp"] <= 1, "cached RoPE bf16 differs by more than 1 ulp"
    if exact:
        assert st["fp8_identical_fraction"] == 1.0 and st["rope_identical"], st
    return st
