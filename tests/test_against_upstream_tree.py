"""Where the upstream source tree is present (the build container; not the GPU box), run its own torch reference
functions on fresh seeded inputs - larger than the committed fixtures - and compare the oracles with them directly.
Skipped elsewhere.  No GPU."""
from __future__ import annotations

import pytest
import torch

from flaggems_vllm.testing import compare, workloads
from oracle import c_oracle, ref_loader, torch_path

pytestmark = pytest.mark.skipif(ref_loader.upstream_root() is None, reason="upstream source tree not present")


@pytest.fixture(scope="module")
def upstream():
    return ref_loader.load_upstream_test_module()


@pytest.mark.parametrize("seed,n,h,bs", [(11, 512, 16, 64), (12, 300, 128, 16), (13, 1000, 1, 64)])
def test_prologue_oracles_against_upstream_ref_impl(upstream, seed, n, h, bs):
    w = workloads.make("long_prefill", device="cpu", seed=seed, num_tokens=n, num_heads=h, num_blocks=(n + bs - 1) // bs + 4)
    nb = w.k_cache.shape[0]
    w.k_cache = w.k_cache[:, : 64 * 584].reshape(-1)[: nb * bs * 584].view(nb, bs * 584).contiguous()
    w.slot_mapping = torch.where(w.slot_mapping >= nb * bs, w.slot_mapping % (nb * bs), w.slot_mapping)
    # slots must stay distinct after the fold
    valid = w.slot_mapping[w.slot_mapping >= 0]
    keep = torch.ones_like(w.slot_mapping, dtype=torch.bool)
    seen = set()
    for i, s in enumerate(w.slot_mapping.tolist()):
        if s >= 0 and s in seen:
            keep[i] = False
        seen.add(s)
    w.slot_mapping = torch.where(keep, w.slot_mapping, torch.full_like(w.slot_mapping, -1))
    cs = upstream.make_cos_sin_cache(131072, 64, torch.float32, "cpu")
    q_up, kc_up = w.q.clone(), w.k_cache.clone()
    upstream.ref_impl(q_up, w.kv.clone(), kc_up, w.slot_mapping.clone(), w.position_ids.clone(), cs, w.eps, bs)
    q_t, kc_t = w.q.clone(), w.k_cache.clone()
    torch_path.prologue(q_t, w.kv, kc_t, w.slot_mapping, w.position_ids, cs, w.eps, bs)
    assert torch.equal(q_t.view(torch.int16), q_up.view(torch.int16)) and torch.equal(kc_t, kc_up)
    q_c, kc_c = w.q.clone(), w.k_cache.clone()
    c_oracle.prologue(q_c, w.kv, kc_c, w.slot_mapping, w.position_ids, cs, w.eps, bs)
    assert torch.equal(kc_c, kc_up)
    st = compare.assert_q_close(q_c, q_up)
    assert st["mismatch_fraction"] < 1e-4
    assert valid.numel() > 0


def test_sibling_oracles_against_upstream_helpers():
    g = torch.Generator().manual_seed(99)
    # weighted RMSNorm
    R = ref_loader.load_upstream_helper_test("test_deepseek_v4_attention_fused_q_kv_rmsnorm.py",
                                             "flaggems_vllm.ops.deepseek_v4_attention_fused_q_kv_rmsnorm", ("fused_q_kv_rmsnorm",))
    x, wgt = torch.randn(200, 1536, generator=g).to(torch.bfloat16), torch.randn(1536, generator=g).to(torch.bfloat16)
    d = compare.bf16_ulp_distance(c_oracle.weighted_rmsnorm(x, wgt, 1e-6), R._rmsnorm_ref(x, wgt, 1e-6))
    assert int(d.max()) <= 1 and float((d != 0).float().mean()) < 1e-3
    # indexer q prologue, both formats
    M = ref_loader.load_upstream_helper_test("test_fused_indexer_q_rope_quant.py", "flaggems_vllm.ops", ("fused_indexer_q_rope_quant",),
                                             package_attrs={"SUPPORTED_FP8_DTYPE": torch.float8_e4m3fn})
    q = (torch.randn(300, 8, 128, generator=g) * torch.logspace(-4, 3, 300)[:, None, None]).to(torch.bfloat16)
    pos = torch.randint(0, 4096, (300,), generator=g)
    cs = M._make_cos_sin_cache(4096, 64, "cpu", torch.float32)
    wts = torch.randn(300, 8, generator=g).to(torch.bfloat16)
    q_rot = M._rotate_tail_gptj(q, pos, cs)
    f8, w8 = M._reference_fp8(q_rot.clone(), wts, 0.09, 0.35)
    out, _, w_out = c_oracle.indexer_q_rope_quant(pos, q, cs, wts, 0.09, 0.35)
    assert torch.equal(out, f8.view(torch.uint8)) and torch.equal(w_out, w8)
    (p4, s4), w4 = M._reference_mxfp4(q_rot.clone(), wts, 0.09, 0.35)
    out, sc, w_out = c_oracle.indexer_q_rope_quant(pos, q, cs, wts, 0.09, 0.35, use_fp4=True)
    assert torch.equal(out, p4) and torch.equal(sc.view(torch.int32).squeeze(-1), s4) and torch.equal(w_out, w4)
    # reader of the indexer key cache
    C = ref_loader.load_upstream_helper_test("test_cp_gather_indexer_k_quant_cache.py", "flaggems_vllm.ops", ("cp_gather_indexer_k_quant_cache",))
    seq_lens = [37, 0, 5, 64, 129] + [3] * 20
    table, cu, blocks = C._make_gather_metadata(seq_lens, 16, "cpu")
    cache = C._make_cache(blocks, 16, 128, 128, torch.float8_e4m3fn, "cpu")
    tokens = int(cu[-1]) + 4
    want_k, want_s = torch.full((tokens, 128), 0x7B, dtype=torch.uint8), torch.full((tokens, 4), 0x7B, dtype=torch.uint8)
    C.torch_gather(cache, want_k.view(torch.float8_e4m3fn), want_s, table, cu)
    got_k, got_s = torch.full_like(want_k, 0x7B), torch.full_like(want_s, 0x7B)
    c_oracle.cp_gather_indexer_k_quant_cache(cache, got_k, got_s, table, cu)
    assert torch.equal(got_k, want_k) and torch.equal(got_s, want_s)


def test_index_oracles_pass_the_upstream_tests():
    """The upstream tests of the two index operators compute their expected values inline, so the oracles are bound in
    the operators' place and the upstream test functions are run on fresh seeded inputs."""
    g = torch.Generator().manual_seed(77)
    G = ref_loader.load_upstream_helper_test(
        "test_deepseek_v4_attention_compute_global_topk_indices_and_lens.py",
        "flaggems_vllm.ops.deepseek_v4_attention_compute_global_topk_indices_and_lens", ("compute_global_topk_indices_and_lens",),
        op_bindings={"compute_global_topk_indices_and_lens": c_oracle.compute_global_topk_indices_and_lens})
    local = torch.randint(-20, 640, (25, 48), generator=g, dtype=torch.int32).clamp(min=-1)
    G.test_compute_global_topk_indices_and_lens_accuracy(
        local.tolist(), torch.randint(0, 3, (25,), generator=g).tolist(), torch.randperm(30, generator=g).view(3, 10).tolist(),
        (torch.rand(25, generator=g) < 0.6).int().tolist(), 64)
    C = ref_loader.load_upstream_helper_test("test_deepseek_v4_attention_combine_topk_swa_indices.py", "flaggems_vllm.ops",
                                             ("combine_topk_swa_indices",),
                                             op_bindings={"combine_topk_swa_indices": c_oracle.combine_topk_swa_indices})
    C.test_combine_topk_swa_indices_accuracy(torch.randint(0, 900, (30, 32), generator=g, dtype=torch.int32).tolist(), [4, 14, 15, 34],
                                             [50, 1, 33], [20, 1, 30], 16, 4, 32, 1000, 200)


def test_prologue_oracles_against_the_upstream_flash_mla_cache_builder():
    """A second, independent statement of the cache format and of the UE8M0 quantiser lives in the upstream FlashMLA
    test (tests/test_flash_mla_with_kvcache.py:94-140, `generate_model1_fp8_kv_cache`).  It draws its own keys; the
    same draws are repeated here, pushed through the oracles with an identity rotation, and the caches compared."""
    F = ref_loader.load_upstream_helper_test("test_flash_mla_with_kvcache.py", "flaggems_vllm.ops.flash_mla_with_kvcache",
                                             ("FlashMLASchedMeta", "flash_mla_with_kvcache", "get_mla_metadata"))
    pages, bs = 5, 64
    torch.manual_seed(123)
    want = F.generate_model1_fp8_kv_cache(pages, bs, device="cpu").view(pages, bs * 584)
    torch.manual_seed(123)
    nope = torch.randn(pages * bs, 448, dtype=torch.bfloat16) * 0.1
    rope = torch.randn(pages * bs, 64, dtype=torch.bfloat16) * 0.1
    kv = torch.cat([nope, rope], dim=1).contiguous()
    n = pages * bs
    table = torch.cat([torch.ones(4, 32), torch.zeros(4, 32)], dim=1).contiguous()  # cos = 1, sin = 0: rotation is the identity
    for run in (c_oracle.prologue, torch_path.prologue):
        q = torch.randn(n, 1, 512).to(torch.bfloat16)
        cache = torch.zeros(pages, bs * 584, dtype=torch.uint8)
        run(q, kv, cache, torch.arange(n), torch.zeros(n, dtype=torch.int64), table, 1e-6, bs)
        assert torch.equal(cache, want)


def test_top_k_oracle_against_upstream_torch_statements():
    """`_torch_topk_ref` (decode) and `reference_top_k_per_row` (prefill) of the upstream tests on fresh logits, compared
    the way those tests compare: the selected values of every row as a sorted list."""
    import types

    runtime = types.SimpleNamespace(torch_device_fn=types.SimpleNamespace(is_available=lambda: True, device_count=lambda: 1))
    D = ref_loader.load_upstream_helper_test("test_top_k_per_row_decode.py", "flaggems_vllm.ops.top_k_per_row_decode", ("top_k_per_row_decode",),
                                             package_attrs={"runtime": runtime})
    P = ref_loader.load_upstream_helper_test("test_top_k_per_row_prefill.py", "flaggems_vllm.ops.top_k_per_row_prefill", ("top_k_per_row_prefill",),
                                             package_attrs={"runtime": runtime})
    g = torch.Generator().manual_seed(55)
    logits = torch.randn(6, 20000, generator=g)
    logits[0, :9000] = 0.5
    seq = torch.tensor([20000, 15000, 300], dtype=torch.int32)
    ref, got = torch.zeros(6, 256, dtype=torch.int32), torch.zeros(6, 256, dtype=torch.int32)
    D._torch_topk_ref(logits.clone(), 2, seq, ref, 6, logits.stride(0), 1, 256)
    c_oracle.top_k_per_row_decode(logits, 2, seq, got, 6, logits.stride(0), 1, 256)
    assert D.check_topk_values_match(logits, got, ref, 256)
    starts = torch.tensor([0, 5, 1000, 19000, 7, 7], dtype=torch.int32)
    ends = torch.tensor([20000, 105, 18000, 20000, 7, 9000], dtype=torch.int32)
    ref = P.reference_top_k_per_row(logits.clone(), starts, ends, 256)
    c_oracle.top_k_per_row_prefill(logits, starts, ends, got, 6, logits.stride(0), 1, 256)
    assert P.check_topk_values_match(logits, got, ref, starts, 256)


def test_group_quant_oracle_against_upstream_torch_statement():
    M = ref_loader.load_upstream_helper_test(
        "test_per_token_group_quant_fp8.py", "flaggems_vllm.ops", ("per_token_group_quant_fp8",),
        sibling_modules={"accuracy_utils": {"FP8_QUANT_SHAPES": {"SEEDS": [0], "GROUP_SIZE": [64], "DTYPES": [torch.bfloat16], "D": [512], "NUM_TOKENS": [7]},
                                            "to_reference": lambda t: t, "gems_assert_close": None, "to_cpu": lambda a, b: a}})
    g = torch.Generator().manual_seed(66)
    x = (torch.randn(50, 2048, generator=g) * torch.logspace(-13, 3, 50)[:, None]).to(torch.bfloat16)
    for group in (64, 128, 256, 512):
        for ue8m0 in (False, True):
            want_q, want_s = M.native_per_token_group_quant_fp8(x, group, dtype=torch.float8_e4m3fn, scale_ue8m0=ue8m0)
            q, s = c_oracle.per_token_group_quant_fp8(x, group, scale_ue8m0=ue8m0)
            assert torch.equal(q, want_q.view(torch.uint8)) and torch.equal(s.view(torch.int32), want_s.view(torch.int32))


def test_act_quant_oracle_against_upstream_torch_statement():
    M = ref_loader.load_upstream_helper_test("test_act_quant.py", "flaggems_vllm.ops", ("act_quant_triton",),
                                             sibling_modules={"accuracy_utils": {"TO_CPU": False, "gems_assert_close": None}})
    g = torch.Generator().manual_seed(67)
    x = (torch.randn(60, 1024, generator=g) * torch.logspace(-8, 3, 60)[:, None]).to(torch.bfloat16)
    for block in (64, 128):
        for fmt in (None, "ue8m0"):
            want_q, want_s = M.torch_act_quant(x, block_size=block, scale_fmt=fmt)
            q, s = c_oracle.act_quant(x, block, fmt)
            assert torch.equal(q, want_q.view(torch.uint8)) and torch.equal(s.view(torch.int32), want_s.view(torch.int32))
