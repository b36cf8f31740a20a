"""`cp_gather_indexer_k_quant_cache`: oracle vs vectors from the upstream test's torch statement; CUDA kernel vs both,
outputs compared bit for bit including the rows no request covers (the upstream bar: rtol=0, atol=0, sentinel rows)."""
from __future__ import annotations

import math

import numpy as np
import pytest
import torch

import flaggems_vllm
from conftest import GOLDEN
from oracle import c_oracle

NAMES = sorted(p.stem for p in GOLDEN.glob("cp_gather_*.npz"))
DEV = "cuda:0"
SENTINEL = 0x7B


def load(name):
    z = np.load(GOLDEN / f"{name}.npz")
    return {k: torch.from_numpy(z[k].copy()) for k in ("cache", "block_table", "cu_seqlen", "k", "scale")}


def metadata(seq_lens, block_size, generator, spare_blocks=3):
    """cu_seqlen, a block table over randomly permuted blocks (-1 where unused), number of blocks."""
    cu = torch.zeros(len(seq_lens) + 1, dtype=torch.int32)
    cu[1:] = torch.cumsum(torch.tensor(seq_lens, dtype=torch.int32), 0)
    per_seq = [math.ceil(n / block_size) for n in seq_lens]
    blocks = sum(per_seq) + spare_blocks
    perm = torch.randperm(blocks, generator=generator).to(torch.int32)
    table = torch.full((len(seq_lens), max(max(per_seq), 1)), -1, dtype=torch.int32)
    at = 0
    for b, n in enumerate(per_seq):
        table[b, :n] = perm[at : at + n]
        at += n
    return cu, table, blocks


def test_golden_files_exist():
    assert len(NAMES) >= 3


@pytest.mark.parametrize("name", NAMES)
def test_oracle_reproduces_upstream_reference(name):
    g = load(name)
    k, scale = torch.full_like(g["k"], SENTINEL), torch.full_like(g["scale"], SENTINEL)
    c_oracle.cp_gather_indexer_k_quant_cache(g["cache"], k, scale, g["block_table"], g["cu_seqlen"])
    assert torch.equal(k, g["k"]) and torch.equal(scale, g["scale"])


@pytest.mark.gpu
@pytest.mark.parametrize("name", NAMES)
def test_kernel_reproduces_upstream_reference(name):
    g = load(name)
    k = torch.full_like(g["k"], SENTINEL).to(DEV).view(torch.float8_e4m3fn)
    scale = torch.full_like(g["scale"], SENTINEL).to(DEV)
    flaggems_vllm.cp_gather_indexer_k_quant_cache(g["cache"].to(DEV), k, scale, g["block_table"].to(DEV), g["cu_seqlen"].to(DEV))
    assert torch.equal(k.view(torch.uint8).cpu(), g["k"]) and torch.equal(scale.cpu(), g["scale"])


@pytest.mark.gpu
@pytest.mark.parametrize("requests,max_len,bs,hd,qbs,extra", [
    (1, 1, 16, 128, 128, 0), (1, 700, 64, 128, 128, 2), (3, 40, 8, 128, 128, 0), (15, 90, 64, 128, 128, 7), (16, 33, 16, 512, 128, 1),
    (17, 50, 64, 128, 128, 0), (31, 20, 4, 64, 32, 3), (127, 9, 64, 128, 128, 5), (128, 9, 64, 128, 16, 0), (300, 12, 16, 256, 64, 9),
    (40, 30, 64, 1024, 128, 0), (9, 25, 12, 96, 48, 4), (11, 19, 16, 120, 24, 2), (5, 40, 16, 192, 64, 1),
])
def test_kernel_matches_oracle(requests, max_len, bs, hd, qbs, extra):
    """Few and many requests (the request of a token is found by bisection; 2^k - 1 requests need the last step),
    empty requests, head sizes on the vector path and off it, more groups than lanes per token, spare output rows."""
    g = torch.Generator().manual_seed(requests * 1000 + hd + qbs)
    seq_lens = torch.randint(0, max_len + 1, (requests,), generator=g).tolist()
    seq_lens[0] = max_len
    cu, table, blocks = metadata(seq_lens, bs, g)
    row = hd + 4 * (hd // qbs)
    cache = torch.randint(0, 256, (blocks, bs, row), generator=g, dtype=torch.uint8)
    tokens = int(cu[-1]) + extra
    want_k = torch.full((tokens, hd), SENTINEL, dtype=torch.uint8)
    want_s = torch.full((tokens, row - hd), SENTINEL, dtype=torch.uint8)
    c_oracle.cp_gather_indexer_k_quant_cache(cache, want_k, want_s, table, cu)
    k, s = torch.full_like(want_k, SENTINEL).to(DEV), torch.full_like(want_s, SENTINEL).to(DEV)
    flaggems_vllm.cp_gather_indexer_k_quant_cache(cache.to(DEV), k, s, table.to(DEV), cu.to(DEV))
    assert torch.equal(k.cpu(), want_k) and torch.equal(s.cpu(), want_s)


@pytest.mark.gpu
def test_float32_scale_tensor_and_padded_rows():
    """Scales handed over as float32 [T, groups] and outputs that are column slices of wider tensors."""
    g = torch.Generator().manual_seed(11)
    cu, table, blocks = metadata([70, 0, 45, 130], 64, g)
    cache = torch.randint(0, 256, (blocks, 64, 132), generator=g, dtype=torch.uint8)
    tokens = int(cu[-1])
    want_k, want_s = torch.zeros(tokens, 128, dtype=torch.uint8), torch.zeros(tokens, 4, dtype=torch.uint8)
    c_oracle.cp_gather_indexer_k_quant_cache(cache, want_k, want_s, table, cu)
    k_wide = torch.zeros(tokens, 256, dtype=torch.uint8, device=DEV)
    s_wide = torch.zeros(tokens, 4, dtype=torch.float32, device=DEV)
    flaggems_vllm.cp_gather_indexer_k_quant_cache(cache.to(DEV), k_wide[:, 128:], s_wide[:, 1:2], table.to(DEV), cu.to(DEV))
    assert torch.equal(k_wide[:, 128:].cpu(), want_k) and not k_wide[:, :128].any()
    assert torch.equal(s_wide[:, 1:2].contiguous().view(torch.uint8).cpu(), want_s) and not s_wide[:, 0].any() and not s_wide[:, 2:].any()


@pytest.mark.gpu
def test_round_trip_with_the_writer():
    """Keys quantised into the cache by indexer_k_quant_and_cache come back, in request order, as the bytes and
    scales the oracle of the writer produced for them."""
    g = torch.Generator().manual_seed(12)
    seq_lens = [200, 64, 1, 333]
    cu, table, blocks = metadata(seq_lens, 64, g)
    tokens = int(cu[-1])
    k = torch.randn(tokens, 128, generator=g).to(torch.bfloat16)
    slots = torch.empty(tokens, dtype=torch.int64)
    for b, n in enumerate(seq_lens):
        off = torch.arange(n)
        slots[int(cu[b]) : int(cu[b + 1])] = table[b, off // 64].to(torch.int64) * 64 + off % 64
    cache = torch.zeros(blocks, 64, 132, dtype=torch.uint8, device=DEV)
    flaggems_vllm.indexer_k_quant_and_cache(k.to(DEV), cache, slots.to(DEV), 128, "ue8m0")
    got_k = torch.empty(tokens, 128, dtype=torch.float8_e4m3fn, device=DEV)
    got_s = torch.empty(tokens, 1, dtype=torch.float32, device=DEV)
    flaggems_vllm.cp_gather_indexer_k_quant_cache(cache, got_k, got_s, table.to(DEV), cu.to(DEV))
    # the writer's oracle on a dense one-token-per-slot cache gives the expected bytes and scales per token
    dense = torch.zeros(1, tokens, 132, dtype=torch.uint8)
    c_oracle.indexer_k_quant_and_cache(k, dense, torch.arange(tokens), 128, "ue8m0")
    flat = dense.view(-1)
    assert torch.equal(got_k.view(torch.uint8).cpu(), flat[: tokens * 128].view(tokens, 128))
    assert torch.equal(got_s.cpu().view(torch.uint8), flat[tokens * 128 :].view(tokens, 4))


def test_host_checks_without_gpu():
    cache = torch.zeros(2, 16, 132, dtype=torch.uint8)
    k, s = torch.zeros(4, 128, dtype=torch.uint8), torch.zeros(4, 4, dtype=torch.uint8)
    table, cu = torch.zeros(1, 1, dtype=torch.int32), torch.tensor([0, 4], dtype=torch.int32)
    with pytest.raises(AssertionError, match="no CPU path"):
        flaggems_vllm.cp_gather_indexer_k_quant_cache(cache, k, s, table, cu)
    with pytest.raises(ValueError):
        flaggems_vllm.cp_gather_indexer_k_quant_cache(cache, torch.zeros(4, 100, dtype=torch.uint8), torch.zeros(4, 12, dtype=torch.uint8), table, cu)
