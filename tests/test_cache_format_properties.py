"""Properties of the prologue's KV path that hold for any input, checked on the C oracle with generated cases (CPU) and,
on fixed cases, on the CUDA kernel: they pin down the cache format independently of any stored vector."""
from __future__ import annotations

import pytest
import torch
from hypothesis import given, settings
from hypothesis import strategies as st

from flaggems_vllm.testing import workloads
from oracle import c_oracle

BS = 16
TABLE = workloads.cos_sin_table(256)


BACKEND = {"device": None}  # None: the C oracle; "cuda:0": the CUDA kernel through the Python entry point


def run(kv, slots, positions, blocks=4, fill=0x5A):
    n = kv.shape[0]
    cache = torch.full((blocks, BS * 584), fill, dtype=torch.uint8)
    q = torch.ones(n, 1, 512, dtype=torch.bfloat16)
    dev = BACKEND["device"]
    if dev is None:
        c_oracle.prologue(q, kv, cache, slots, positions, TABLE, 1e-6, BS)
        return cache
    import flaggems_vllm

    cache = cache.to(dev)
    flaggems_vllm.fused_deepseek_v4_qnorm_rope_kv_rope_quant_insert(q.to(dev), kv.to(dev), cache, slots.to(dev), positions.to(dev), TABLE.to(dev), 1e-6, BS)
    return cache.cpu()


def records(cache, slots):
    """(576 data bytes, 8 scale bytes) of every slot >= 0, in the order given."""
    out = []
    for s in slots.tolist():
        if s < 0:
            continue
        block, pos = divmod(s, BS)
        row = cache[block]
        out.append((row[pos * 576 : (pos + 1) * 576].clone(), row[BS * 576 + pos * 8 : BS * 576 + (pos + 1) * 8].clone()))
    return out


cases = st.tuples(st.integers(1, 12), st.integers(0, 2**31 - 1))


def make(n, seed, spread=True):
    g = torch.Generator().manual_seed(seed)
    scale = torch.logspace(-3, 2, n)[:, None] if spread else 1.0
    kv = (torch.randn(n, 512, generator=g) * scale).to(torch.bfloat16)
    slots = torch.randperm(4 * BS, generator=g)[:n].to(torch.int64)
    positions = torch.randint(0, 256, (n,), generator=g, dtype=torch.int64)
    return kv, slots, positions


@settings(max_examples=25, deadline=None)
@given(cases, st.integers(-6, 6))
def test_power_of_two_input_scaling_moves_only_the_scale_codes(case, shift):
    """kv * 2^j: every UE8M0 code moves by j, the e4m3 bytes stay (the quantiser sees the same mantissas); the rotated bf16
    tail scales exactly."""
    kv, slots, positions = make(*case)
    scaled = (kv.float() * 2.0**shift).to(torch.bfloat16)  # exact: a power of two
    a, b = records(run(kv, slots, positions), slots), records(run(scaled, slots, positions), slots)
    for (data_a, scale_a), (data_b, scale_b) in zip(a, b):
        codes_a, codes_b = scale_a[:7].to(torch.int32), scale_b[:7].to(torch.int32)
        floor = 127 + torch.ceil(torch.log2(torch.tensor(1e-4 / 448.0))).int()  # groups below the amax clamp keep the clamp's code
        free = (codes_a > floor) & (codes_b > floor)
        assert torch.equal((codes_b - codes_a)[free], torch.full_like(codes_a, shift)[free])
        for g in range(7):
            if bool(free[g]):
                assert torch.equal(data_a[64 * g : 64 * (g + 1)], data_b[64 * g : 64 * (g + 1)])
        tail_a = data_a[448:].view(torch.bfloat16).float() * 2.0**shift
        assert torch.equal(tail_a.to(torch.bfloat16), data_b[448:].view(torch.bfloat16))
        assert int(scale_a[7]) == 0 and int(scale_b[7]) == 0


@settings(max_examples=25, deadline=None)
@given(cases)
def test_a_record_depends_only_on_its_token(case):
    """Permuting the tokens together with their slots and positions gives the same cache; every record equals the record
    the token gets when it is inserted alone."""
    kv, slots, positions = make(*case)
    n = kv.shape[0]
    perm = torch.randperm(n, generator=torch.Generator().manual_seed(case[1] ^ 1))
    whole = run(kv, slots, positions)
    assert torch.equal(whole, run(kv[perm].contiguous(), slots[perm].contiguous(), positions[perm].contiguous()))
    t = int(perm[0])
    alone = run(kv[t : t + 1].contiguous(), slots[t : t + 1].contiguous(), positions[t : t + 1].contiguous())
    (da, sa), (db, sb) = records(whole, slots[t : t + 1])[0], records(alone, slots[t : t + 1])[0]
    assert torch.equal(da, db) and torch.equal(sa, sb)


@settings(max_examples=25, deadline=None)
@given(cases, st.integers(0, 255))
def test_skipped_tokens_and_free_slots_keep_their_bytes(case, fill):
    """Slot -1 and tokens beyond len(slot_mapping) write nothing; bytes of slots that no token maps to keep the fill."""
    kv, slots, positions = make(*case)
    n = kv.shape[0]
    keep = max(1, n - 2)
    masked = slots[:keep].clone()
    masked[::3] = -1
    cache = run(kv, masked, positions, fill=fill)
    touched = torch.zeros(4, BS * 584, dtype=torch.bool)
    for s in masked.tolist():
        if s >= 0:
            block, pos = divmod(s, BS)
            touched[block, pos * 576 : (pos + 1) * 576] = True
            touched[block, BS * 576 + pos * 8 : BS * 576 + (pos + 1) * 8] = True
    assert bool((cache[~touched] == fill).all())


@settings(max_examples=15, deadline=None)
@given(cases)
def test_reader_inverts_the_quantiser_within_half_a_step(case):
    """De-quantising the record gives back every unrotated value within half an e4m3 step at its group's scale, and the
    rotated tail exactly as stored."""
    kv, slots, positions = make(*case, spread=False)
    cache = run(kv, slots, positions)
    back = c_oracle.gather_dequant(cache, slots, BS).float()
    for t in range(kv.shape[0]):
        (_, scale) = records(cache, slots[t : t + 1])[0]
        for g in range(7):
            step = 2.0 ** (int(scale[g]) - 127)
            x, y = kv[t, 64 * g : 64 * (g + 1)].float(), back[t, 64 * g : 64 * (g + 1)]
            # e4m3 keeps 4 significant bits: the error is at most 1/16 of the value's power of two, in units of the scale; bf16 rounding of the product adds 2^-8
            bound = torch.maximum(x.abs() / 16.0, torch.tensor(step * 2.0**-10)) * 1.01 + x.abs() * 2.0**-8
            assert bool(((x - y).abs() <= bound).all())


@pytest.mark.gpu
@pytest.mark.parametrize("n,seed", [(1, 1), (5, 2), (12, 3), (9, 4)])
def test_the_same_properties_hold_for_the_cuda_kernel(n, seed):
    BACKEND["device"] = "cuda:0"
    try:
        test_power_of_two_input_scaling_moves_only_the_scale_codes.hypothesis.inner_test((n, seed), 3)
        test_power_of_two_input_scaling_moves_only_the_scale_codes.hypothesis.inner_test((n, seed), -5)
        test_a_record_depends_only_on_its_token.hypothesis.inner_test((n, seed))
        test_skipped_tokens_and_free_slots_keep_their_bytes.hypothesis.inner_test((n, seed), 0xA7)
        kv, slots, positions = make(n, seed, spread=False)
        on_device = run(kv, slots, positions)
        BACKEND["device"] = None
        assert torch.equal(on_device, run(kv, slots, positions))
    finally:
        BACKEND["device"] = None
