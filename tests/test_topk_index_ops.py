"""`compute_global_topk_indices_and_lens` and `combine_topk_swa_indices`: oracle vs vectors that passed the upstream
tests' own expected-value code; CUDA kernels vs both, every int32 compared (the upstream bar: exact equality)."""
from __future__ import annotations

import numpy as np
import pytest
import torch

import flaggems_vllm
from conftest import GOLDEN
from oracle import c_oracle

GLOBAL = sorted(p.stem for p in GOLDEN.glob("global_topk_*.npz"))
COMBINE = sorted(p.stem for p in GOLDEN.glob("combine_topk_swa_*.npz"))
DEV = "cuda:0"
UNWRITTEN = -77


def load(name):
    z = np.load(GOLDEN / f"{name}.npz")
    return {k: (torch.from_numpy(z[k].copy()) if z[k].ndim else int(z[k])) for k in z.files}


def test_golden_files_exist():
    assert len(GLOBAL) >= 5 and len(COMBINE) >= 5


@pytest.mark.parametrize("name", GLOBAL)
def test_global_topk_oracle_reproduces_upstream_expectation(name):
    g = load(name)
    out, lens = c_oracle.compute_global_topk_indices_and_lens(g["topk_indices"], g["token_to_req"], g["block_table"], g["block_size"], g["is_valid"])
    assert torch.equal(out, g["global_indices"]) and torch.equal(lens, g["lens"])


@pytest.mark.parametrize("name", COMBINE)
def test_combine_oracle_reproduces_upstream_expectation(name):
    g = load(name)
    out, lens = c_oracle.combine_topk_swa_indices(g["topk_indices"], g["query_start_loc"], g["seq_lens"], g["gather_lens"], g["window_size"],
                                                  g["compress_ratio"], g["topk"], g["M"], g["N"])
    assert torch.equal(out, g["combined"]) and torch.equal(lens, g["lens"])


@pytest.mark.gpu
@pytest.mark.parametrize("name", GLOBAL)
def test_global_topk_kernel_reproduces_upstream_expectation(name):
    g = load(name)
    out, lens = flaggems_vllm.compute_global_topk_indices_and_lens(g["topk_indices"].to(DEV), g["token_to_req"].to(DEV), g["block_table"].to(DEV),
                                                                   g["block_size"], g["is_valid"].to(DEV))
    assert out.dtype == torch.int32 and lens.dtype == torch.int32
    assert torch.equal(out.cpu(), g["global_indices"]) and torch.equal(lens.cpu(), g["lens"])


@pytest.mark.gpu
@pytest.mark.parametrize("name", COMBINE)
def test_combine_kernel_reproduces_upstream_expectation(name):
    g = load(name)
    out, lens = flaggems_vllm.combine_topk_swa_indices(g["topk_indices"].to(DEV), g["query_start_loc"].to(DEV), g["seq_lens"].to(DEV),
                                                       g["gather_lens"].to(DEV), g["window_size"], g["compress_ratio"], g["topk"], g["M"], g["N"])
    assert out.shape == g["combined"].shape and out.dtype == torch.int32
    assert torch.equal(out.cpu(), g["combined"]) and torch.equal(lens.cpu(), g["lens"])


@pytest.mark.gpu
@pytest.mark.parametrize("tokens,topk,reqs,blocks,bs,valid", [
    (1, 4, 1, 2, 4, True), (300, 512, 7, 40, 64, True), (129, 2048, 5, 300, 64, False), (50, 100, 3, 9, 16, True),
    (33, 37, 2, 11, 12, True), (64, 1024, 64, 16, 256, False), (10, 132, 2, 50, 3, True),
])
def test_global_topk_kernel_matches_oracle(tokens, topk, reqs, blocks, bs, valid):
    """Vector rows (topk % 4 == 0) and scalar ones, block sizes that are and are not powers of two, with and without
    the validity vector, a row slice of a wider tensor as input."""
    g = torch.Generator().manual_seed(tokens + topk + bs)
    wide = torch.randint(0, blocks * bs, (tokens, topk + 8), generator=g, dtype=torch.int32)
    wide[torch.rand(tokens, topk + 8, generator=g) < 0.25] = -1
    local = wide[:, 4 : 4 + topk]
    req = torch.randint(0, reqs, (tokens,), generator=g, dtype=torch.int32)
    table = torch.randint(0, 1 << 20, (reqs, blocks), generator=g, dtype=torch.int32)
    is_valid = (torch.rand(tokens, generator=g) < 0.8).to(torch.int32) if valid else None
    want, want_lens = c_oracle.compute_global_topk_indices_and_lens(local.contiguous(), req, table, bs, is_valid)
    got, got_lens = flaggems_vllm.compute_global_topk_indices_and_lens(wide.to(DEV)[:, 4 : 4 + topk], req.to(DEV), table.to(DEV), bs,
                                                                       None if is_valid is None else is_valid.to(DEV))
    assert torch.equal(got.cpu(), want) and torch.equal(got_lens.cpu(), want_lens)


@pytest.mark.gpu
@pytest.mark.parametrize("query_lens,window,ratio,topk,width,m,n", [
    ([1], 128, 4, 512, 512, 8192, 2048), ([40, 1, 77, 3], 128, 4, 512, 512, 8192, 2048), ([5] * 31, 8, 2, 16, 16, 100, 30),
    ([9, 0, 4], 5, 3, 6, 9, 50, 7), ([300], 128, 4, 2048, 2048, 65536, 4096), ([17, 23], 100, 128, 10, 12, 500, 100),
])
def test_combine_kernel_matches_oracle(query_lens, window, ratio, topk, width, m, n):
    """One and many requests (an empty one, 2^k - 1 of them), short and long histories, vector and scalar rows, spare
    rows behind the last request that must stay unwritten."""
    g = torch.Generator().manual_seed(sum(query_lens) + window + topk)
    tokens = sum(query_lens)
    spare = 3
    start = torch.tensor([7] + (7 + torch.cumsum(torch.tensor(query_lens), 0)).tolist(), dtype=torch.int32)
    seq = torch.tensor([q + int(torch.randint(0, 4 * window + 2, (1,), generator=g)) for q in query_lens], dtype=torch.int32)
    gather = torch.minimum(seq, torch.tensor(query_lens, dtype=torch.int32) + window)
    values = torch.randint(0, m, (tokens + spare, width), generator=g, dtype=torch.int32)
    want, want_lens = c_oracle.combine_topk_swa_indices(values, start, seq, gather, window, ratio, topk, m, n, fill=UNWRITTEN)
    got, got_lens = flaggems_vllm.combine_topk_swa_indices(values.to(DEV), start.to(DEV), seq.to(DEV), gather.to(DEV), window, ratio, topk, m, n)
    assert torch.equal(got.cpu()[:tokens], want[:tokens]) and torch.equal(got_lens.cpu()[:tokens], want_lens[:tokens])
    assert bool((want[tokens:] == UNWRITTEN).all())  # the oracle leaves uncovered rows alone too


@pytest.mark.gpu
def test_index_operators_feed_the_cache_reader():
    """End to end over the paged cache: slots from compute_global_topk_indices_and_lens address the same tokens the
    prologue wrote (slot = block * block_size + offset is the slot_mapping convention)."""
    g = torch.Generator().manual_seed(5)
    bs, blocks_per_req = 64, 6
    table = torch.randperm(2 * blocks_per_req, generator=g).to(torch.int32).view(2, blocks_per_req)
    local = torch.randint(0, bs * blocks_per_req, (8, 16), generator=g, dtype=torch.int32)
    req = torch.tensor([0, 0, 1, 1, 0, 1, 0, 1], dtype=torch.int32)
    slots, lens = flaggems_vllm.compute_global_topk_indices_and_lens(local.to(DEV), req.to(DEV), table.to(DEV), bs)
    want = table[req.long()[:, None], (local // bs).long()] * bs + local % bs
    assert torch.equal(slots.cpu(), want) and bool((lens.cpu() == 16).all())


def test_host_checks_without_gpu():
    idx = torch.zeros(2, 4, dtype=torch.int32)
    with pytest.raises(AssertionError, match="no CPU path"):
        flaggems_vllm.compute_global_topk_indices_and_lens(idx, torch.zeros(2, dtype=torch.int32), torch.zeros(1, 1, dtype=torch.int32), 4)
    with pytest.raises(AssertionError, match="no CPU path"):
        flaggems_vllm.combine_topk_swa_indices(idx, torch.tensor([0, 2], dtype=torch.int32), torch.tensor([2], dtype=torch.int32),
                                               torch.tensor([2], dtype=torch.int32), 4, 2, 4, 64, 16)
    with pytest.raises(AssertionError):
        flaggems_vllm.compute_global_topk_indices_and_lens(torch.zeros(4, dtype=torch.int32), None, None, 4)
