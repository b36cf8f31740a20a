"""Writes the golden vectors under tests/golden/ by running the UPSTREAM torch reference.

    python tests/golden/make_golden.py          # needs the upstream tree (see oracle/ref_loader.py)

Every case feeds seeded inputs to the upstream test file's own `ref_impl`
(tests/test_fused_deepseek_v4_qnorm_rope_kv_rope_quant_insert.py:316-333) on CPU and
stores inputs and outputs (bf16 as uint16 bit patterns) in one compressed .npz per case.
The upstream tree is not available where the GPU tests run, so the vectors are committed.
`cpu_ref` (256 tokens x 8 heads) stores its inputs' SHA-256 instead of the 2 MiB q tensor:
inputs are regenerated from the seed by flaggems_vllm.testing.workloads and the test checks
the digest before trusting the comparison.
"""
from __future__ import annotations

import hashlib
import sys
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent
ROOT = HERE.parent.parent
sys.path[:0] = [str(ROOT), str(ROOT / "flaggems-vllm_b200")]

from oracle import ref_loader  # noqa: E402
from flaggems_vllm.testing import workloads  # noqa: E402

TOKEN_BYTES = 584


def u16(t: torch.Tensor) -> np.ndarray:
    return t.contiguous().view(torch.int16).numpy().view(np.uint16)


def sha(t: torch.Tensor) -> str:
    return hashlib.sha256(t.contiguous().view(torch.uint8).numpy().tobytes()).hexdigest()


def case_inputs(name: str):
    """(q, kv, k_cache, slot_mapping, positions, max_pos, block_size) for the small stored cases."""
    g = torch.Generator().manual_seed({"q_path": 0, "kv_path_bs16": 1, "kv_path_bs64": 1, "dp_padding": 3,
                                       "mixed": 5, "edge_rows": 6, "padded_stride": 7}[name])
    rn = lambda *s: torch.randn(*s, generator=g).to(torch.bfloat16)  # noqa: E731
    if name == "q_path":  # T:358-402 shape family: kv zero, every slot -1
        n, h, bs, nb = 17, 8, 16, 2
        return rn(n, h, 512), torch.zeros(n, 512, dtype=torch.bfloat16), torch.zeros(nb, bs * TOKEN_BYTES, dtype=torch.uint8), \
            torch.full((n,), -1, dtype=torch.int64), torch.arange(n), 4096, bs
    if name in ("kv_path_bs16", "kv_path_bs64"):  # T:419-462
        bs = 16 if name.endswith("16") else 64
        n = 17 if bs == 16 else 64
        nb = (n + bs - 1) // bs + 1
        return torch.zeros(n, 1, 512, dtype=torch.bfloat16), rn(n, 512), torch.zeros(nb, bs * TOKEN_BYTES, dtype=torch.uint8), \
            torch.arange(n), torch.arange(n), 4096, bs
    if name == "dp_padding":  # T:468-515: slot_mapping shorter than q
        n, pad, bs = 17, 5, 16
        nb = (n + bs - 1) // bs + 1
        return torch.zeros(n + pad, 1, 512, dtype=torch.bfloat16), rn(n + pad, 512), \
            torch.zeros(nb, bs * TOKEN_BYTES, dtype=torch.uint8), torch.arange(n), torch.arange(n + pad), 4096, bs
    if name == "mixed":  # what upstream never tests: random positions, scattered slots, -1 among them, dirty cache
        n, h, bs, nb = 33, 8, 16, 6
        slots = torch.randperm(nb * bs, generator=g)[:n]
        slots[torch.randperm(n, generator=g)[:6]] = -1
        return rn(n, h, 512), rn(n, 512), torch.randint(0, 256, (nb, bs * TOKEN_BYTES), generator=g, dtype=torch.uint8), \
            slots, torch.randint(0, 4096, (n,), generator=g), 4096, bs
    if name == "edge_rows":  # quantisation corner cases in kv; q rows with extreme norms
        n, h, bs, nb = 32, 2, 16, 3
        q, kv = rn(n, h, 512), rn(n, 512)
        kvf = kv.float()
        kvf[0] = 0.0                                    # all-zero groups: amax clamps to 1e-4
        kvf[1] *= 1e-5                                  # below the clamp
        kvf[2] *= 1e4                                   # large
        kvf[3] *= 50.0                                  # outlier row
        for k in range(4, 20):                          # amax = 7 * 2^k exactly -> amax/448 is a power of two
            kvf[k, :448] = kvf[k, :448].clamp(-1, 1)
            kvf[k, 5:448:64] = 7.0 * 2.0 ** (k - 12)
            kvf[k, :448] = kvf[k, :448].clamp(-7.0 * 2.0 ** (k - 12), 7.0 * 2.0 ** (k - 12))
        kvf[20, :448] = 448.0                            # scale exactly 1, every value saturates the format top
        kvf[21, :448] = -448.0
        kvf[22, :448:2] = 1e-4                           # exactly at the clamp
        kvf[23, :448] = torch.linspace(-3, 3, 448)      # ties and subnormals after scaling
        kvf[24, :448] = torch.linspace(-0.02, 0.02, 448)
        kvf[24, 7] = 3.5
        qf = q.float()
        qf[0] = 0.0                                     # zero row: rsqrt(eps)
        qf[1] *= 1e-3
        qf[2] *= 50.0
        qf[3] *= 1e4
        return qf.to(torch.bfloat16), kvf.to(torch.bfloat16), \
            torch.randint(0, 256, (nb, bs * TOKEN_BYTES), generator=g, dtype=torch.uint8), \
            torch.randperm(nb * bs, generator=g)[:n], torch.randint(0, 4096, (n,), generator=g), 4096, bs
    if name == "padded_stride":  # block pitch larger than bs*584 (and 16-byte aligned): a strided view
        n, h, bs, nb = 20, 3, 16, 4
        slots = torch.randperm(nb * bs, generator=g)[:n]
        slots[3] = -1
        return rn(n, h, 512), rn(n, 512), torch.randint(0, 256, (nb, bs * TOKEN_BYTES + 64), generator=g, dtype=torch.uint8), \
            slots, torch.randint(0, 4096, (n,), generator=g), 4096, bs
    raise KeyError(name)


SMALL_CASES = ("q_path", "kv_path_bs16", "kv_path_bs64", "dp_padding", "mixed", "edge_rows", "padded_stride")


def main() -> None:
    T = ref_loader.load_upstream_test_module()
    for name in SMALL_CASES:
        q, kv, kc, slots, pos, max_pos, bs = case_inputs(name)
        slots, pos = slots.to(torch.int64), pos.to(torch.int64)
        cs = T.make_cos_sin_cache(max_pos, 64, torch.float32, "cpu")  # theta 10000 for max_pos <= 8192
        q_out, kv_work, kc_out = q.clone(), kv.clone(), kc.clone()
        T.ref_impl(q_out, kv_work, kc_out, slots.clone(), pos.clone(), cs.clone(), 1e-6, bs)
        np.savez_compressed(
            HERE / f"{name}.npz", q=u16(q), kv=u16(kv), k_cache=kc.numpy(), slot_mapping=slots.numpy(),
            position_ids=pos.numpy(), max_pos=max_pos, block_size=bs, eps=1e-6, q_out=u16(q_out), k_cache_out=kc_out.numpy(),
        )
        print(name, "ok")

    # benchmark configuration "CPU torch reference path, seed 0": digest-checked regenerated inputs
    w = workloads.make("cpu_ref", device="cpu", seed=0)
    cs_up = T.make_cos_sin_cache(4096, 64, torch.float32, "cpu")
    assert torch.equal(cs_up, w.cos_sin_cache), "workload cos/sin table differs from the upstream helper"
    q_out, kc_out = w.q.clone(), w.k_cache.clone()
    T.ref_impl(q_out, w.kv.clone(), kc_out, w.slot_mapping.clone(), w.position_ids.clone(), w.cos_sin_cache.clone(),
               w.eps, w.cache_block_size)
    blk, off = w.slot_mapping // 64, w.slot_mapping % 64
    data = kc_out.view(64, -1)[:, : 64 * 576].reshape(64, 64, 576)[blk, off]
    scales = kc_out.view(64, -1)[:, 64 * 576 :].reshape(64, 64, 8)[blk, off]
    np.savez_compressed(
        HERE / "cpu_ref.npz",
        input_sha=np.array([sha(w.q), sha(w.kv), sha(w.k_cache), sha(w.slot_mapping), sha(w.position_ids)]),
        q_out_head=u16(q_out[:48]), q_out_sha=sha(q_out), k_cache_out_sha=sha(kc_out),
        rows_data=data.numpy(), rows_scales=scales.numpy(), torch_version=torch.__version__,
    )
    print("cpu_ref ok")


def gather_cases() -> None:
    """Known-answer vectors of the cache reader, built with the upstream test's own `_fill_cache`
    (tests/test_deepseek_v4_attention_dequantize_and_gather_k_cache.py:42-63) and the parameter sets of
    its accuracy test (:66-119): hand-made cache rows and the rows they must de-quantise to."""
    G = ref_loader.load_upstream_helper_test(
        "test_deepseek_v4_attention_dequantize_and_gather_k_cache.py",
        "flaggems_vllm.ops.deepseek_v4_attention_dequantize_and_gather_k_cache", ("dequantize_and_gather_k_cache",))
    for batch, seq_len, gather_len, block_size, nope_dim, rope_dim in ((1, 6, 3, 4, 64, 16), (2, 12, 5, 64, 448, 64),
                                                                        (3, 150, 70, 64, 448, 64)):
        scale_slots = (nope_dim + 63) // 64 + (1 if nope_dim % 64 == 0 else 0)
        token_data = nope_dim + rope_dim * 2
        blocks_per_seq = (seq_len + block_size - 1) // block_size
        num_blocks = batch * blocks_per_seq
        k_cache = torch.zeros(num_blocks, block_size * (token_data + scale_slots), dtype=torch.uint8)
        expected = torch.zeros(batch, gather_len, nope_dim + rope_dim, dtype=torch.bfloat16)
        rows = {}
        for req in range(batch):
            for i in range(gather_len):
                pos = seq_len - gather_len + i
                slot = (req * blocks_per_seq + pos // block_size) * block_size + pos % block_size
                rows[slot] = expected[req : req + 1, i : i + 1, :]
        G._fill_cache(k_cache, rows, block_size, nope_dim, rope_dim, scale_slots)
        np.savez_compressed(
            HERE / f"gather_b{batch}_s{seq_len}_g{gather_len}_bs{block_size}_n{nope_dim}_r{rope_dim}.npz",
            k_cache=k_cache.numpy(), expected=u16(expected), seq_lens=np.full(batch, seq_len, np.int32),
            gather_lens=np.full(batch, gather_len, np.int32),
            block_table=np.arange(num_blocks, dtype=np.int32).reshape(batch, blocks_per_seq), block_size=block_size,
            nope_dim=nope_dim, rope_dim=rope_dim, scale_slots=scale_slots)
        print("gather", batch, seq_len, gather_len, block_size, nope_dim, rope_dim, "ok")


def rmsnorm_cases() -> None:
    """Seeded inputs through the upstream test's own torch reference `_rmsnorm_ref`
    (tests/test_deepseek_v4_attention_fused_q_kv_rmsnorm.py:40-44), at its two shapes (:47-53) plus one
    with row strides and values of mixed magnitude."""
    R = ref_loader.load_upstream_helper_test(
        "test_deepseek_v4_attention_fused_q_kv_rmsnorm.py", "flaggems_vllm.ops.deepseek_v4_attention_fused_q_kv_rmsnorm",
        ("fused_q_kv_rmsnorm",))
    for idx, (tokens, qdim, kvdim) in enumerate(((4, 256, 128), (8, 1536, 512), (33, 1536, 512))):
        g = torch.Generator().manual_seed(100 + idx)
        rn = lambda *s: torch.randn(*s, generator=g).to(torch.bfloat16)  # noqa: E731
        qr, kv, qw, kw = rn(tokens, qdim), rn(tokens, kvdim), rn(qdim), rn(kvdim)
        if idx == 2:
            qr = (qr.float() * torch.logspace(-3, 3, tokens)[:, None]).to(torch.bfloat16)
            kv[0] = 0
        np.savez_compressed(HERE / f"rmsnorm_t{tokens}_q{qdim}_kv{kvdim}.npz", qr=u16(qr), kv=u16(kv), q_weight=u16(qw),
                            kv_weight=u16(kw), eps=1e-6, q_out=u16(R._rmsnorm_ref(qr, qw, 1e-6)),
                            kv_out=u16(R._rmsnorm_ref(kv, kw, 1e-6)))
        print("rmsnorm", tokens, qdim, kvdim, "ok")


def inv_rope_cases() -> None:
    """Seeded inputs through the upstream test's torch statement `native_fused_inv_rope_fp8_quant`
    (tests/test_fused_inv_rope_fp8_quant.py:150-198), both scale formats, its head/group shapes (:104-115),
    a x1000 saturation case (:430-442) and rows built to hit exact powers of two."""
    shapes = {"NUM_TOKENS": [7], "NUM_HEADS_AND_GROUPS": [(64, 8)], "OUTPUT_LAYOUT_NUM_TOKENS": [7],
              "OUTPUT_LAYOUT_NUM_HEADS_AND_GROUPS": [(64, 8)], "PER_GROUP_CONTIGUITY_NUM_TOKENS": [7],
              "REAL_ROPE_NUM_TOKENS": [32], "TMA_ALIGNED_SCALES": [False, True], "SEEDS": [0, 42]}
    M = ref_loader.load_upstream_helper_test(
        "test_fused_inv_rope_fp8_quant.py", "flaggems_vllm.ops", ("per_token_group_quant_fp8", "fused_inv_rope_fp8_quant"),
        package_attrs={"SUPPORTED_FP8_DTYPE": torch.float8_e4m3fn},
        sibling_modules={"accuracy_utils": {"FUSED_INV_ROPE_FP8_QUANT_SHAPES": shapes}})
    cs = M._make_cos_sin_cache(4096, 64, "cpu")
    for idx, (tokens, heads, groups, scale) in enumerate(((3, 64, 8, 1.0), (1, 32, 4, 1.0), (5, 16, 2, 1000.0), (6, 8, 8, 1.0))):
        g = torch.Generator().manual_seed(200 + idx)
        o = (scale * torch.randn(tokens, heads, 512, generator=g)).to(torch.bfloat16)
        if idx == 3:  # exact powers of two, zero groups, tiny groups
            of = o.float()
            of[0, 0, :128] = 0.0
            of[0, 1, :128] *= 1e-12
            for k in range(2, 8):
                of[0, k, :128] = of[0, k, :128].clamp(-1, 1)
                of[0, k, 5] = 1.75 * 2.0 ** (k - 4)
            o = of.to(torch.bfloat16)
        pos = torch.randint(0, 4096, (tokens,), generator=g)
        out = {}
        for packed in (False, True):
            f8, sc = M.native_fused_inv_rope_fp8_quant(o, pos, cs, groups, heads // groups, tma_aligned_scales=packed)
            out[f"fp8_{int(packed)}"] = f8.view(torch.uint8).numpy()
            out[f"scale_{int(packed)}"] = sc.numpy()
        np.savez_compressed(HERE / f"inv_rope_t{tokens}_h{heads}_g{groups}.npz", o=u16(o), positions=pos.numpy(), n_groups=groups,
                            heads_per_group=heads // groups, **out)
        print("inv_rope", tokens, heads, groups, "ok")


def indexer_cases() -> None:
    """Seeded inputs through the upstream test's torch statement `torch_indexer` and its cache builder
    (tests/test_indexer_k_quant_and_cache.py:99-171), at the test's parameter sets (:174-181) plus fp32-scale ones."""
    M = ref_loader.load_upstream_helper_test("test_indexer_k_quant_and_cache.py", "flaggems_vllm.ops", ("indexer_k_quant_and_cache",))
    cases = ((torch.bfloat16, 19, 4, 16, 128, 128, "ue8m0"), (torch.float16, 23, 5, 16, 512, 128, "ue8m0"),
             (torch.bfloat16, 17, 4, 64, 512, 128, "ue8m0"), (torch.bfloat16, 21, 3, 16, 128, 128, "fp32"),
             (torch.float16, 9, 2, 8, 256, 64, "fp32"))
    for idx, (dtype, tokens, blocks, bs, hd, qbs, fmt) in enumerate(cases):
        torch.manual_seed(300 + idx)
        k = torch.randn(tokens, hd, dtype=dtype)
        if idx == 3:
            k[0] = 0
            k[1] *= 1e-6
            k[2, 5] = 1.75 * 4
        slots = M._make_slot_mapping(tokens, blocks, bs, "cpu")
        cache = M._make_cache(blocks, bs, hd, qbs, "cpu")
        out = cache.clone()
        M.torch_indexer(k, out, slots, qbs, fmt)
        name = f"indexer_{'f16' if dtype == torch.float16 else 'bf16'}_t{tokens}_b{blocks}x{bs}_d{hd}_q{qbs}_{fmt}"
        np.savez_compressed(HERE / f"{name}.npz", k=u16(k), is_fp16=int(dtype == torch.float16), slot_mapping=slots.numpy(),
                            cache=cache.numpy(), cache_out=out.numpy(), quant_block_size=qbs, scale_fmt=fmt)
        print(name, "ok")


def indexer_q_cases() -> None:
    """Seeded inputs through the upstream test's torch statements `_rotate_tail_gptj`, `_reference_fp8` and
    `_reference_mxfp4` (tests/test_fused_indexer_q_rope_quant.py:48-113), with the test's geometry (8 heads x 128,
    rotary tail 64, fp32 and bf16 tables) and its token counts (:121)."""
    M = ref_loader.load_upstream_helper_test("test_fused_indexer_q_rope_quant.py", "flaggems_vllm.ops", ("fused_indexer_q_rope_quant",),
                                             package_attrs={"SUPPORTED_FP8_DTYPE": torch.float8_e4m3fn})
    for tokens in (1, 7, 32):
        for cache_dtype in (torch.float32, torch.bfloat16):
            torch.manual_seed(400 + tokens)
            q = torch.randn(tokens, 8, 128, dtype=torch.bfloat16)
            if tokens == 7:  # zero head, tiny head, exact power-of-two amax, e2m1 ties
                q[0, 0] = 0
                q[0, 1] *= 1e-6
                q[1, 0, :64] = torch.tensor([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, 6.0] * 8).to(torch.bfloat16)
                q[1, 1, 3] = 7.0
            pos = torch.randint(0, 4096, (tokens,), dtype=torch.int64)
            cs = M._make_cos_sin_cache(4096, 64, "cpu", cache_dtype)
            w = torch.randn(tokens, 8, dtype=torch.bfloat16)
            sm, hs = 128 ** -0.5, 8 ** -0.5
            q_rot = M._rotate_tail_gptj(q, pos, cs)
            f8, w8 = M._reference_fp8(q_rot.clone(), w, sm, hs)
            (p4, s4), w4 = M._reference_mxfp4(q_rot.clone(), w, sm, hs)
            name = f"indexer_q_t{tokens}_{'bf16' if cache_dtype == torch.bfloat16 else 'f32'}table"
            np.savez_compressed(HERE / f"{name}.npz", q=u16(q), positions=pos.numpy(), weights=u16(w), table_bf16=int(cache_dtype == torch.bfloat16),
                                fp8=f8.view(torch.uint8).numpy(), w_fp8=w8.numpy(), fp4=p4.numpy(), fp4_scales=s4.numpy(), w_fp4=w4.numpy())
            print(name, "ok")


def cp_gather_cases() -> None:
    """Seeded caches and request metadata from the upstream test's own builders through its torch statement
    `torch_gather` (tests/test_cp_gather_indexer_k_quant_cache.py:85-171), at the test's two parameter sets (:176-179)
    plus a case with more than 16 requests, one of them empty."""
    M = ref_loader.load_upstream_helper_test("test_cp_gather_indexer_k_quant_cache.py", "flaggems_vllm.ops",
                                             ("cp_gather_indexer_k_quant_cache",))
    cases = (([13, 7, 16], 8, 128, 128, 0), ([17, 1, 33, 9], 16, 512, 128, 5),
             ([3, 9, 1, 12, 0, 8, 2, 7, 11, 4, 6, 10, 1, 3, 9, 2, 5, 7, 4, 8, 6, 1, 13, 2, 3, 5, 4, 9, 7, 6, 2], 4, 64, 32, 3))
    for idx, (seq_lens, bs, hd, qbs, extra) in enumerate(cases):
        torch.manual_seed(500 + idx)
        table, cu, blocks = M._make_gather_metadata(seq_lens, bs, "cpu")
        perm = torch.randperm(blocks, dtype=torch.int32)  # scatter the blocks, which the upstream builder leaves in order
        table = torch.where(table >= 0, perm[table.clamp(min=0).long()], table)
        cache = M._make_cache(blocks, bs, hd, qbs, torch.float8_e4m3fn, "cpu")
        tokens = int(cu[-1]) + extra
        k = torch.full((tokens, hd), 0x7B, dtype=torch.uint8)
        scale = torch.full((tokens, hd * 4 // qbs), 0x7B, dtype=torch.uint8)
        M.torch_gather(cache, k.view(torch.float8_e4m3fn), scale, table, cu)
        name = f"cp_gather_r{len(seq_lens)}_b{bs}_d{hd}_q{qbs}_x{extra}"
        np.savez_compressed(HERE / f"{name}.npz", cache=cache.numpy(), block_table=table.numpy(), cu_seqlen=cu.numpy(),
                            k=k.numpy(), scale=scale.numpy(), quant_block_size=qbs)
        print(name, "ok")


def flash_mla_builder_case() -> None:
    """A cache made by the independent statement of the format and quantiser in the upstream FlashMLA test
    (`generate_model1_fp8_kv_cache`, tests/test_flash_mla_with_kvcache.py:94-140), with the keys it drew
    (same seed, same order of draws: 448 unrotated values, then the 64 rotary ones, both randn * 0.1)."""
    F = ref_loader.load_upstream_helper_test("test_flash_mla_with_kvcache.py", "flaggems_vllm.ops.flash_mla_with_kvcache",
                                             ("FlashMLASchedMeta", "flash_mla_with_kvcache", "get_mla_metadata"))
    pages, bs = 3, 16
    torch.manual_seed(700)
    cache = F.generate_model1_fp8_kv_cache(pages, bs, device="cpu").view(pages, bs * 584)
    torch.manual_seed(700)
    nope = torch.randn(pages * bs, 448, dtype=torch.bfloat16) * 0.1
    rope = torch.randn(pages * bs, 64, dtype=torch.bfloat16) * 0.1
    np.savez_compressed(HERE / "flash_mla_builder_cache.npz", kv=u16(torch.cat([nope, rope], dim=1).contiguous()), cache=cache.numpy(),
                        block_size=bs)
    print("flash_mla_builder_cache ok")


def topk_cases() -> None:
    """Seeded logits through the upstream tests' torch statements `_torch_topk_ref`
    (tests/test_top_k_per_row_decode.py:111-124) and `reference_top_k_per_row` (tests/test_top_k_per_row_prefill.py:80-99).
    Stored: logits, ranges, and the SORTED VALUES the reference selected per row (its tests compare selected values, not
    positions: ties are broken arbitrarily), with -inf where a row has fewer than top_k valid entries."""
    D = ref_loader.load_upstream_helper_test("test_top_k_per_row_decode.py", "flaggems_vllm.ops.top_k_per_row_decode", ("top_k_per_row_decode",),
                                             package_attrs={"runtime": types_namespace()})
    P = ref_loader.load_upstream_helper_test("test_top_k_per_row_prefill.py", "flaggems_vllm.ops.top_k_per_row_prefill", ("top_k_per_row_prefill",),
                                             package_attrs={"runtime": types_namespace()})

    def selected_values(logits, idx, starts):
        out = torch.full(idx.shape, float("-inf"))
        for r in range(idx.shape[0]):
            valid = idx[r][idx[r] >= 0].long() + int(starts[r])
            out[r, : valid.numel()] = logits[r, valid].sort(descending=True).values
        return out

    gen = torch.Generator().manual_seed(800)
    for idx_case, (rows, vocab, top_k, next_n) in enumerate(((3, 700, 64, 1), (4, 3000, 512, 2), (2, 5000, 128, 1))):
        logits = torch.randn(rows, vocab, generator=gen)
        if idx_case == 2:  # many ties and a block of near-equal values (low 8 bits only differ)
            logits[0, :3000] = 1.5
            logits[1] = (0x3F900000 | torch.randint(0, 256, (vocab,), generator=gen, dtype=torch.int32)).view(torch.float32)
        seq = torch.randint(top_k // 2, vocab, (-(-rows // next_n),), generator=gen, dtype=torch.int32)
        ref = torch.zeros(rows, top_k, dtype=torch.int32)
        D._torch_topk_ref(logits.clone(), next_n, seq, ref, rows, logits.stride(0), logits.stride(1), top_k)
        np.savez_compressed(HERE / f"topk_decode_{idx_case}.npz", logits=logits.numpy(), seq_lens=seq.numpy(), next_n=next_n, top_k=top_k,
                            values=selected_values(logits, ref, torch.zeros(rows)).numpy())
        print("topk_decode", idx_case, "ok")
    for idx_case, (rows, vocab, top_k) in enumerate(((5, 900, 64), (4, 257, 512), (6, 4000, 256))):
        logits = torch.randn(rows, vocab, generator=gen)
        starts = torch.randint(0, vocab // 2, (rows,), generator=gen, dtype=torch.int32)
        ends = torch.minimum(starts + torch.randint(1, vocab, (rows,), generator=gen, dtype=torch.int32), torch.tensor(vocab, dtype=torch.int32))
        ref = P.reference_top_k_per_row(logits.clone(), starts, ends, top_k)
        np.savez_compressed(HERE / f"topk_prefill_{idx_case}.npz", logits=logits.numpy(), row_starts=starts.numpy(), row_ends=ends.numpy(),
                            top_k=top_k, values=selected_values(logits, ref, starts).numpy())
        print("topk_prefill", idx_case, "ok")


def types_namespace():
    import types

    return types.SimpleNamespace(torch_device_fn=types.SimpleNamespace(is_available=lambda: True, device_count=lambda: 1))


def group_quant_cases() -> None:
    """Seeded activations through the upstream test's torch statement `native_per_token_group_quant_fp8`
    (tests/test_per_token_group_quant_fp8.py:53-89), at the test's group sizes (64 ... 512), both scale formats, with the
    test's uniform inputs and with normal ones that include a zero group, a tiny group and an exact-power-of-two maximum."""
    M = ref_loader.load_upstream_helper_test("test_per_token_group_quant_fp8.py", "flaggems_vllm.ops", ("per_token_group_quant_fp8",),
                                             sibling_modules={"accuracy_utils": {"FP8_QUANT_SHAPES": {"SEEDS": [0], "GROUP_SIZE": [64], "DTYPES": [torch.bfloat16], "D": [512], "NUM_TOKENS": [7]},
                                                                                 "to_reference": lambda t: t, "gems_assert_close": None, "to_cpu": lambda a, b: a}})
    idx = 0
    for tokens, cols, group in ((7, 512, 64), (7, 512, 128), (5, 1024, 256), (3, 1024, 512)):
        for ue8m0 in (False, True):
            torch.manual_seed(900 + idx)
            x = torch.rand(tokens, cols, dtype=torch.bfloat16) if idx % 4 < 2 else torch.randn(tokens, cols).to(torch.bfloat16)
            x[0, :group] = 0
            x[1, :group] *= 1e-12
            x[2, 0] = 448.0
            q, sc = M.native_per_token_group_quant_fp8(x, group, dtype=torch.float8_e4m3fn, scale_ue8m0=ue8m0)
            np.savez_compressed(HERE / f"group_quant_t{tokens}_k{cols}_g{group}_{'ue8m0' if ue8m0 else 'fp32'}.npz", x=u16(x), group_size=group,
                                ue8m0=int(ue8m0), bytes=q.view(torch.uint8).numpy(), scales=sc.numpy())
            print("group_quant", tokens, cols, group, ue8m0, "ok")
            idx += 1


def act_quant_cases() -> None:
    """Seeded activations through the upstream test's torch statement `torch_act_quant` (tests/test_act_quant.py:49-99)."""
    M = ref_loader.load_upstream_helper_test("test_act_quant.py", "flaggems_vllm.ops", ("act_quant_triton",),
                                             sibling_modules={"accuracy_utils": {"TO_CPU": False, "gems_assert_close": None}})
    idx = 0
    for rows, cols, block in ((40, 128, 128), (7, 896, 64), (5, 2048, 128)):
        for fmt in (None, "ue8m0"):
            torch.manual_seed(950 + idx)
            x = torch.randn(rows, cols).to(torch.bfloat16)
            x[0, :block] = 0
            x[1, :block] *= 1e-6
            x[2, 0] = 448.0
            y, sc = M.torch_act_quant(x, block_size=block, scale_fmt=fmt)
            np.savez_compressed(HERE / f"act_quant_m{rows}_n{cols}_b{block}_{fmt or 'fp32'}.npz", x=u16(x), block_size=block, round_scale=int(fmt is not None),
                                bytes=y.view(torch.uint8).numpy(), scales=sc.numpy())
            print("act_quant", rows, cols, block, fmt, "ok")
            idx += 1


def _parameter_sets(test_function):
    return [m for m in test_function.pytestmark if m.name == "parametrize"][0].args[1]


def index_cases() -> None:
    """The two index operators of the sparse attention.  Their upstream tests compute the expected values inline
    (tests/test_deepseek_v4_attention_compute_global_topk_indices_and_lens.py:92-111,
    tests/test_deepseek_v4_attention_combine_topk_swa_indices.py:129-155), so each case is RUN THROUGH THE UPSTREAM
    TEST FUNCTION with the oracle bound in the operator's place: the function returns only if its own expected values
    equal the oracle's output, which is then stored.  Cases: the tests' parameter sets and seeded larger ones."""
    from oracle import c_oracle

    G = ref_loader.load_upstream_helper_test(
        "test_deepseek_v4_attention_compute_global_topk_indices_and_lens.py",
        "flaggems_vllm.ops.deepseek_v4_attention_compute_global_topk_indices_and_lens", ("compute_global_topk_indices_and_lens",),
        op_bindings={"compute_global_topk_indices_and_lens": c_oracle.compute_global_topk_indices_and_lens})
    check = G.test_compute_global_topk_indices_and_lens_accuracy
    cases = [tuple(a) for a in _parameter_sets(check)]
    gen = torch.Generator().manual_seed(600)
    for tokens, topk, reqs, blocks_per_req, bs in ((9, 12, 3, 5, 4), (17, 128, 4, 9, 64), (6, 33, 2, 7, 12)):
        local = torch.randint(0, blocks_per_req * bs, (tokens, topk), generator=gen, dtype=torch.int32)
        local[torch.rand(tokens, topk, generator=gen) < 0.3] = -1
        local[0] = -1
        table = torch.randperm(reqs * blocks_per_req, generator=gen).to(torch.int32).view(reqs, blocks_per_req)
        cases.append((local.tolist(), torch.randint(0, reqs, (tokens,), generator=gen).tolist(), table.tolist(),
                      (torch.rand(tokens, generator=gen) < 0.7).int().tolist(), bs))
    for idx, (local, req, table, valid, bs) in enumerate(cases):
        check(local, req, table, valid, bs)  # raises if the oracle differs from the upstream expectation
        t = lambda v: torch.tensor(v, dtype=torch.int32)
        out, lens = c_oracle.compute_global_topk_indices_and_lens(t(local), t(req), t(table), bs, t(valid))
        np.savez_compressed(HERE / f"global_topk_{idx}.npz", topk_indices=t(local).numpy(), token_to_req=t(req).numpy(),
                            block_table=t(table).numpy(), is_valid=t(valid).numpy(), block_size=bs, global_indices=out.numpy(),
                            lens=lens.numpy())
        print("global_topk", idx, "ok")

    C = ref_loader.load_upstream_helper_test("test_deepseek_v4_attention_combine_topk_swa_indices.py", "flaggems_vllm.ops",
                                             ("combine_topk_swa_indices",),
                                             op_bindings={"combine_topk_swa_indices": c_oracle.combine_topk_swa_indices})
    check = C.test_combine_topk_swa_indices_accuracy
    cases = [tuple(a) for a in _parameter_sets(check)]
    gen = torch.Generator().manual_seed(601)
    for query_lens, window, ratio, topk, width, m, n in (([5, 1, 9], 8, 4, 16, 16, 300, 40), ([3, 7, 2, 12], 128, 4, 64, 64, 4096, 1024),
                                                         ([20], 5, 3, 6, 9, 50, 7)):
        tokens = sum(query_lens)
        start = [100] + (100 + torch.cumsum(torch.tensor(query_lens), 0)).tolist()  # a non-zero first entry is subtracted
        seq = [q + int(torch.randint(0, 60, (1,), generator=gen)) for q in query_lens]
        gather = [min(s, q + int(torch.randint(0, 30, (1,), generator=gen))) for s, q in zip(seq, query_lens)]
        cases.append((torch.randint(0, m - 1, (tokens, width), generator=gen, dtype=torch.int32).tolist(), start, seq, gather, window,
                      ratio, topk, m, n))
    for idx, (values, start, seq, gather, window, ratio, topk, m, n) in enumerate(cases):
        check(values, start, seq, gather, window, ratio, topk, m, n)
        t = lambda v: torch.tensor(v, dtype=torch.int32)
        combined, lens = c_oracle.combine_topk_swa_indices(t(values), t(start), t(seq), t(gather), window, ratio, topk, m, n)
        np.savez_compressed(HERE / f"combine_topk_swa_{idx}.npz", topk_indices=t(values).numpy(), query_start_loc=t(start).numpy(),
                            seq_lens=t(seq).numpy(), gather_lens=t(gather).numpy(), window_size=window, compress_ratio=ratio, topk=topk,
                            M=m, N=n, combined=combined.numpy(), lens=lens.numpy())
        print("combine_topk_swa", idx, "ok")


if __name__ == "__main__":
    if len(sys.argv) < 2 or sys.argv[1] == "flash_mla":
        flash_mla_builder_case()
    if len(sys.argv) < 2 or sys.argv[1] == "act_quant":
        act_quant_cases()
    if len(sys.argv) < 2 or sys.argv[1] == "group_quant":
        group_quant_cases()
    if len(sys.argv) < 2 or sys.argv[1] == "topk":
        topk_cases()
    if len(sys.argv) < 2 or sys.argv[1] == "index":
        index_cases()
    if len(sys.argv) < 2 or sys.argv[1] == "cp_gather":
        cp_gather_cases()
    if len(sys.argv) < 2 or sys.argv[1] == "indexer_q":
        indexer_q_cases()
    if len(sys.argv) < 2 or sys.argv[1] == "indexer":
        indexer_cases()
    if len(sys.argv) < 2 or sys.argv[1] == "inv_rope":
        inv_rope_cases()
    if len(sys.argv) < 2 or sys.argv[1] == "rmsnorm":
        rmsnorm_cases()
    if len(sys.argv) < 2 or sys.argv[1] == "prologue":
        main()
    if len(sys.argv) < 2 or sys.argv[1] == "gather":
        gather_cases()
