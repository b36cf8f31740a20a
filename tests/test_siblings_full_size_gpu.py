"""The sibling operators at the sizes `bench.py` times them at, compared in full with their oracles."""
from __future__ import annotations

import pytest
import torch

import flaggems_vllm
from flaggems_vllm.testing import compare, workloads
from oracle import c_oracle

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def gen(seed):
    return torch.Generator(device=DEV).manual_seed(seed)


@pytest.mark.parametrize("packed", [True, False])
def test_epilogue_quantiser_8192_tokens_128_heads(packed):
    g = gen(1)
    o = torch.randn(8192, 128, 512, generator=g, device=DEV, dtype=torch.float32).to(torch.bfloat16)
    pos = torch.randint(0, 65536, (8192,), generator=g, device=DEV, dtype=torch.int64)
    cs = workloads.cos_sin_table(65536, device=DEV)
    fp8, scale = flaggems_vllm.fused_inv_rope_fp8_quant(o, pos, cs, 8, 16, tma_aligned_scales=packed)
    want_fp8, want_scale = c_oracle.inv_rope_fp8_quant(o.cpu(), pos.cpu(), cs.cpu(), 8, 16, packed=packed)
    assert torch.equal(fp8.cpu().view(torch.uint8), want_fp8)
    assert torch.equal(scale.cpu().contiguous().view(torch.int32), want_scale.view(torch.int32))


@pytest.mark.parametrize("use_fp4", [False, True])
def test_indexer_q_prologue_16384_tokens_64_heads(use_fp4):
    g = gen(2)
    q = torch.randn(16384, 64, 128, generator=g, device=DEV).to(torch.bfloat16)
    pos = torch.randint(0, 65536, (16384,), generator=g, device=DEV, dtype=torch.int64)
    cs = workloads.cos_sin_table(65536, device=DEV)
    w = torch.randn(16384, 64, generator=g, device=DEV).to(torch.bfloat16)
    res, w_out = flaggems_vllm.fused_indexer_q_rope_quant(pos, q, cs, w, 0.0884, 0.125, use_fp4=use_fp4)
    want_q, want_s, want_w = c_oracle.indexer_q_rope_quant(pos.cpu(), q.cpu(), cs.cpu(), w.cpu(), 0.0884, 0.125, use_fp4=use_fp4)
    assert torch.equal(w_out.cpu(), want_w)
    if use_fp4:
        assert torch.equal(res[0].cpu(), want_q) and torch.equal(res[1].cpu().view(torch.uint8).view(16384, 64, 4), want_s)
    else:
        assert torch.equal(res.cpu().view(torch.uint8), want_q)


def test_indexer_k_insert_one_million_tokens():
    g = gen(3)
    n = 1 << 20
    k = torch.randn(n, 128, generator=g, device=DEV).to(torch.bfloat16)
    cache = torch.randint(0, 256, (n // 64 + 8, 64, 132), generator=g, device=DEV, dtype=torch.uint8)
    slots = torch.randperm(cache.shape[0] * 64, generator=g, device=DEV)[:n].to(torch.int64)
    slots[::17] = -1
    want = cache.cpu().clone()
    c_oracle.indexer_k_quant_and_cache(k.cpu(), want, slots.cpu(), 128, "ue8m0")
    flaggems_vllm.indexer_k_quant_and_cache(k, cache, slots, 128, "ue8m0")
    assert torch.equal(cache.cpu(), want)


def test_q_kv_rmsnorm_65536_tokens():
    g = gen(4)
    qr = torch.randn(65536, 1536, generator=g, device=DEV).to(torch.bfloat16)
    kv = torch.randn(65536, 512, generator=g, device=DEV).to(torch.bfloat16)
    qw = (1 + 0.1 * torch.randn(1536, generator=g, device=DEV)).to(torch.bfloat16)
    kw = (1 + 0.1 * torch.randn(512, generator=g, device=DEV)).to(torch.bfloat16)
    q_out, kv_out = flaggems_vllm.fused_q_kv_rmsnorm(qr, kv, qw, kw, 1e-6)
    for got, x, wt in ((q_out, qr, qw), (kv_out, kv, kw)):
        d = compare.bf16_ulp_distance(got.cpu(), c_oracle.weighted_rmsnorm(x.cpu(), wt.cpu(), 1e-6))
        assert int(d.max()) <= 1 and float((d != 0).float().mean()) < 1e-3


def test_cache_reader_262144_tokens():
    g = gen(5)
    reqs, seq, bs = 16, 16384, 64
    blocks = reqs * seq // bs
    cache = torch.randint(0, 256, (blocks, bs * 584), generator=g, device=DEV, dtype=torch.uint8)
    cache[(cache & 0x7F) == 0x7F] = 0x41  # no e4m3 NaN codes
    region = cache[:, bs * 576 :]
    region.copy_(torch.randint(100, 140, region.shape, generator=g, device=DEV, dtype=torch.uint8))
    table = torch.randperm(blocks, generator=g, device=DEV).to(torch.int32).view(reqs, seq // bs).contiguous()
    lens = torch.randint(seq // 2, seq + 1, (reqs,), generator=g, device=DEV, dtype=torch.int32)
    out = torch.zeros(reqs, seq, 512, device=DEV, dtype=torch.bfloat16)
    flaggems_vllm.dequantize_and_gather_k_cache(out, cache, lens, None, table, bs)
    want = torch.zeros(reqs, seq, 512, dtype=torch.bfloat16)
    c_oracle.dequantize_and_gather(want, cache.cpu(), lens.cpu(), None, table.cpu(), bs)
    assert torch.equal(out.cpu().view(torch.int16), want.view(torch.int16))


def test_indexer_cache_reader_one_million_tokens():
    g = gen(6)
    n, reqs, bs = 1 << 20, 16, 64
    cache = torch.randint(0, 256, (n // bs, bs, 132), generator=g, device=DEV, dtype=torch.uint8)
    table = torch.randperm(n // bs, generator=g, device=DEV).to(torch.int32).view(reqs, -1).contiguous()
    lens = torch.randint(n // reqs // 2, n // reqs + 1, (reqs,), generator=g, device=DEV, dtype=torch.int32)
    cu = torch.zeros(reqs + 1, device=DEV, dtype=torch.int32)
    cu[1:] = torch.cumsum(lens, 0)
    tokens = int(cu[-1]) + 5
    k = torch.full((tokens, 128), 0x7B, device=DEV, dtype=torch.uint8)
    s = torch.full((tokens, 4), 0x7B, device=DEV, dtype=torch.uint8)
    flaggems_vllm.cp_gather_indexer_k_quant_cache(cache, k, s, table, cu)
    want_k, want_s = torch.full((tokens, 128), 0x7B, dtype=torch.uint8), torch.full((tokens, 4), 0x7B, dtype=torch.uint8)
    c_oracle.cp_gather_indexer_k_quant_cache(cache.cpu(), want_k, want_s, table.cpu(), cu.cpu())
    assert torch.equal(k.cpu(), want_k) and torch.equal(s.cpu(), want_s)


def test_index_operators_32768_tokens():
    g = gen(7)
    n, reqs = 32768, 16
    local = torch.randint(0, 65536, (n, 2048), generator=g, device=DEV, dtype=torch.int32)
    local[torch.rand(n, 2048, generator=g, device=DEV) < 0.1] = -1
    req = torch.randint(0, reqs, (n,), generator=g, device=DEV, dtype=torch.int32)
    table = torch.randperm(reqs * 1024, generator=g, device=DEV).to(torch.int32).view(reqs, 1024).contiguous()
    valid = (torch.rand(n, generator=g, device=DEV) < 0.9).to(torch.int32)
    got, lens = flaggems_vllm.compute_global_topk_indices_and_lens(local, req, table, 64, valid)
    want, want_lens = c_oracle.compute_global_topk_indices_and_lens(local.cpu(), req.cpu(), table.cpu(), 64, valid.cpu())
    assert torch.equal(got.cpu(), want) and torch.equal(lens.cpu(), want_lens)
    del local, got
    values = torch.randint(0, 8192, (n, 512), generator=g, device=DEV, dtype=torch.int32)
    cg = torch.Generator().manual_seed(7)
    q_lens = torch.randint(1, n // reqs, (reqs,), generator=cg)  # ragged requests; the last one takes the rest
    q_lens[-1] = n - int(q_lens[:-1].sum())
    start = torch.zeros(reqs + 1, dtype=torch.int32)
    start[1:] = torch.cumsum(q_lens, 0)
    seq = (q_lens + torch.randint(0, 3000, (reqs,), generator=cg)).to(torch.int32)
    gather = torch.minimum(seq, (q_lens + 128).to(torch.int32))
    got, lens = flaggems_vllm.combine_topk_swa_indices(values, start.to(DEV), seq.to(DEV), gather.to(DEV), 128, 4, 512, 8192, 2048)
    want, want_lens = c_oracle.combine_topk_swa_indices(values.cpu(), start, seq, gather, 128, 4, 512, 8192, 2048)
    assert torch.equal(got.cpu(), want) and torch.equal(lens.cpu(), want_lens)


@pytest.mark.parametrize("rows,vocab,top_k", [(1, 262144, 512), (496, 262144, 512), (4096, 32768, 2048), (8192, 8192, 512)])
def test_top_k_selection_at_bench_sizes(rows, vocab, top_k):
    """Too large for the sorting oracle on every row: the values selected on every row must equal, as a sorted list, the
    values torch.topk returns on the device (the property the upstream tests check), and 8 rows go through the oracle."""
    g = gen(8)
    logits = torch.randn(rows, vocab, generator=g, device=DEV)
    seq = torch.full((rows,), vocab, device=DEV, dtype=torch.int32)
    idx = torch.full((rows, top_k), -7, device=DEV, dtype=torch.int32)
    flaggems_vllm.top_k_per_row_decode(logits, 1, seq, idx, rows, logits.stride(0), logits.stride(1), top_k)
    assert int(idx.min()) >= 0 and int(idx.max()) < vocab
    got = logits.gather(1, idx.long()).sort(dim=1, descending=True).values
    want = torch.topk(logits, top_k, dim=1, sorted=True).values
    assert torch.equal(got, want)
    assert int((idx.sort(dim=1).values.diff(dim=1) == 0).sum()) == 0  # no position twice
    pick = torch.linspace(0, rows - 1, min(rows, 8)).long()
    sub = logits[pick.to(DEV)].cpu()
    ref = torch.zeros(pick.numel(), top_k, dtype=torch.int32)
    c_oracle.top_k_per_row_decode(sub, 1, torch.full((pick.numel(),), vocab, dtype=torch.int32), ref, pick.numel(), sub.stride(0), 1, top_k)
    assert torch.equal(sub.gather(1, ref.long()).sort(dim=1, descending=True).values, got[pick.to(DEV)].cpu())
