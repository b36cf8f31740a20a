"""`top_k_per_row_decode` / `top_k_per_row_prefill`: oracle vs vectors from the upstream tests' torch statements; CUDA
kernel vs both.  As upstream, what is compared are the selected VALUES of every row as a sorted list (ties may be
broken differently), here exactly rather than within 1e-6; in addition every returned position must be inside the
row's range and distinct, and the tail must be -1."""
from __future__ import annotations

import numpy as np
import pytest
import torch

import flaggems_vllm
from conftest import GOLDEN
from oracle import c_oracle

DECODE = sorted(p.stem for p in GOLDEN.glob("topk_decode_*.npz"))
PREFILL = sorted(p.stem for p in GOLDEN.glob("topk_prefill_*.npz"))
DEV = "cuda:0"


def load(name):
    z = np.load(GOLDEN / f"{name}.npz")
    return {k: (torch.from_numpy(z[k].copy()) if z[k].ndim else int(z[k])) for k in z.files}


def decode_ends(seq_lens, next_n, rows):
    r = torch.arange(rows)
    return (seq_lens.long()[r // next_n] - next_n + r % next_n + 1).clamp(min=0)


def selected_values(logits, indices, starts, ends, top_k):
    """Sorted selected values per row (-inf padding), after checking that the positions are a valid selection."""
    logits, indices = logits.cpu(), indices.cpu()
    out = torch.full(indices.shape, float("-inf"))
    for r in range(indices.shape[0]):
        length = max(0, min(int(ends[r]), logits.shape[1]) - int(starts[r]))
        k = min(top_k, length)
        row = indices[r].long()
        assert bool((row[k:] == -1).all()), "tail must be -1"
        assert bool(((row[:k] >= 0) & (row[:k] < length)).all()), "positions must lie inside the row's range"
        assert row[:k].unique().numel() == k, "positions must be distinct"
        out[r, :k] = logits[r, row[:k] + int(starts[r])].sort(descending=True).values
    return out


def test_golden_files_exist():
    assert len(DECODE) >= 3 and len(PREFILL) >= 3


@pytest.mark.parametrize("name", DECODE)
def test_oracle_reproduces_upstream_decode_reference(name):
    g = load(name)
    rows = g["logits"].shape[0]
    idx = torch.zeros(rows, g["top_k"], dtype=torch.int32)
    c_oracle.top_k_per_row_decode(g["logits"], g["next_n"], g["seq_lens"], idx, rows, g["logits"].stride(0), 1, g["top_k"])
    got = selected_values(g["logits"], idx, torch.zeros(rows), decode_ends(g["seq_lens"], g["next_n"], rows), g["top_k"])
    assert torch.equal(got, g["values"])


@pytest.mark.parametrize("name", PREFILL)
def test_oracle_reproduces_upstream_prefill_reference(name):
    g = load(name)
    rows = g["logits"].shape[0]
    idx = torch.zeros(rows, g["top_k"], dtype=torch.int32)
    c_oracle.top_k_per_row_prefill(g["logits"], g["row_starts"], g["row_ends"], idx, rows, g["logits"].stride(0), 1, g["top_k"])
    assert torch.equal(selected_values(g["logits"], idx, g["row_starts"], g["row_ends"], g["top_k"]), g["values"])


@pytest.mark.gpu
@pytest.mark.parametrize("name", DECODE)
def test_kernel_reproduces_upstream_decode_reference(name):
    g = load(name)
    rows = g["logits"].shape[0]
    logits = g["logits"].to(DEV)
    idx = torch.full((rows, g["top_k"]), 7, dtype=torch.int32, device=DEV)
    flaggems_vllm.top_k_per_row_decode(logits, g["next_n"], g["seq_lens"].to(DEV), idx, rows, logits.stride(0), logits.stride(1), g["top_k"])
    got = selected_values(g["logits"], idx, torch.zeros(rows), decode_ends(g["seq_lens"], g["next_n"], rows), g["top_k"])
    assert torch.equal(got, g["values"])


@pytest.mark.gpu
@pytest.mark.parametrize("name", PREFILL)
def test_kernel_reproduces_upstream_prefill_reference(name):
    g = load(name)
    rows = g["logits"].shape[0]
    logits = g["logits"].to(DEV)
    idx = torch.full((rows, g["top_k"]), 7, dtype=torch.int32, device=DEV)
    flaggems_vllm.top_k_per_row_prefill(logits, g["row_starts"].to(DEV), g["row_ends"].to(DEV), idx, rows, logits.stride(0), logits.stride(1), g["top_k"])
    assert torch.equal(selected_values(g["logits"], idx, g["row_starts"], g["row_ends"], g["top_k"]), g["values"])


def run_both(logits, starts, ends, top_k):
    rows = logits.shape[0]
    want = torch.zeros(rows, top_k, dtype=torch.int32)
    c_oracle.top_k_per_row_prefill(logits, starts, ends, want, rows, logits.stride(0), logits.stride(1), top_k)
    dev = logits.to(DEV)
    got = torch.full((rows, top_k), 7, dtype=torch.int32, device=DEV)
    flaggems_vllm.top_k_per_row_prefill(dev, starts.to(DEV), ends.to(DEV), got, rows, dev.stride(0), dev.stride(1), top_k)
    assert torch.equal(selected_values(logits, got, starts, ends, top_k), selected_values(logits, want, starts, ends, top_k))


@pytest.mark.gpu
@pytest.mark.parametrize("rows,vocab,top_k", [(1, 262144, 512), (8, 129280, 1024), (496, 4096, 64), (3, 32768, 2048), (5, 8192, 256), (2, 1000, 1000), (4, 257, 512)])
def test_kernel_matches_oracle_on_random_logits(rows, vocab, top_k):
    """The upstream shape lists (batch 1 and 496, vocabularies 4096 ... 262144, top_k 64 ... 1024) with ragged ranges."""
    g = torch.Generator().manual_seed(rows + vocab + top_k)
    logits = torch.randn(rows, vocab, generator=g)
    starts = torch.randint(0, vocab // 3, (rows,), generator=g, dtype=torch.int32)
    ends = torch.randint(2 * vocab // 3, vocab + 1, (rows,), generator=g, dtype=torch.int32)
    starts[0], ends[0] = 0, vocab
    run_both(logits, starts, ends, top_k)


@pytest.mark.gpu
@pytest.mark.parametrize("case", ["all_equal", "low_8_bits", "two_values", "with_infinities", "negative_only", "descending_ramp", "tiny_range", "empty_range"])
def test_kernel_on_degenerate_rows(case):
    """Rows that crowd one histogram bin (the slow route), ties across the k-th value, infinities, signed zeros,
    ranges shorter than top_k and empty ranges."""
    g = torch.Generator().manual_seed(1)
    vocab, top_k = 70000, 512
    logits = torch.randn(2, vocab, generator=g)
    starts, ends = torch.zeros(2, dtype=torch.int32), torch.full((2,), vocab, dtype=torch.int32)
    if case == "all_equal":
        logits[0] = 0.25
    elif case == "low_8_bits":  # the upstream test_logits_diff_in_8LSBits
        logits[0] = (0x3F900000 | torch.randint(0, 256, (vocab,), generator=g, dtype=torch.int32)).view(torch.float32)
    elif case == "two_values":
        logits[0] = torch.where(torch.rand(vocab, generator=g) < 0.004, 2.0, 1.0)  # ~280 large ones, the rest tie
    elif case == "with_infinities":
        logits[0, ::1000] = float("inf")
        logits[0, 1::1000] = float("-inf")
        logits[0, 2::1000] = 0.0
        logits[0, 3::1000] = -0.0
    elif case == "negative_only":
        logits[0] = -logits[0].abs() - 1.0
    elif case == "descending_ramp":
        logits[0] = torch.linspace(5.0, -5.0, vocab)
    elif case == "tiny_range":
        starts[0], ends[0] = 100, 130
    elif case == "empty_range":
        starts[0], ends[0] = 500, 500
    run_both(logits, starts, ends, top_k)


@pytest.mark.gpu
def test_decode_rows_share_sequence_lengths_and_strided_logits():
    """next_n = 2: rows 2b and 2b+1 see seq_lens[b] - 1 and seq_lens[b] entries; logits given as a column slice."""
    g = torch.Generator().manual_seed(3)
    wide = torch.randn(6, 9000, generator=g)
    logits = wide[:, 500:8500]
    seq = torch.tensor([8000, 3000, 40], dtype=torch.int32)
    want = torch.zeros(6, 128, dtype=torch.int32)
    c_oracle.top_k_per_row_decode(logits, 2, seq, want, 6, logits.stride(0), logits.stride(1), 128)
    dev = wide.to(DEV)[:, 500:8500]
    got = torch.full((6, 128), 7, dtype=torch.int32, device=DEV)
    flaggems_vllm.top_k_per_row_decode(dev, 2, seq.to(DEV), got, 6, dev.stride(0), dev.stride(1), 128)
    ends = decode_ends(seq, 2, 6)
    assert torch.equal(selected_values(logits, got, torch.zeros(6), ends, 128), selected_values(logits, want, torch.zeros(6), ends, 128))


@pytest.mark.gpu
@pytest.mark.parametrize("lengths,k,two_d", [([70000, 512, 100, 65536, 0, 33000], 512, False), ([32773, 32774], 1024, True), ([262144] * 3, 2048, False)])
def test_persistent_topk_call_shape(lengths, k, two_d):
    """vLLM's `persistent_topk(logits, lengths, output, workspace, k, max_seq_len)`: rows padded with -inf as in the
    upstream test, lengths 1-D or [batch, next_n], the workspace left untouched."""
    g = torch.Generator().manual_seed(len(lengths) + k)
    width = max(max(lengths), k) + 64
    logits = torch.full((len(lengths), width), float("-inf"))
    for r, n in enumerate(lengths):
        logits[r, :n] = torch.randn(n, generator=g)
    lens = torch.tensor(lengths, dtype=torch.int32)
    want = torch.zeros(len(lengths), k, dtype=torch.int32)
    c_oracle.top_k_per_row_prefill(logits, torch.zeros(len(lengths), dtype=torch.int32), lens, want, len(lengths), logits.stride(0), 1, k)
    got = torch.full((len(lengths), k), 7, dtype=torch.int32, device=DEV)
    workspace = torch.full((1 << 16,), 0x5A, dtype=torch.uint8, device=DEV)
    flaggems_vllm.persistent_topk(logits.to(DEV), (lens.view(1, -1) if two_d else lens).to(DEV), got, workspace, k=k, max_seq_len=max(lengths))
    starts = torch.zeros(len(lengths))
    assert torch.equal(selected_values(logits, got, starts, lens, k), selected_values(logits, want, starts, lens, k))
    assert bool((workspace == 0x5A).all())


@pytest.mark.gpu
@pytest.mark.parametrize("layout", ["odd_offset", "odd_row_stride", "transposed"])
def test_rows_that_are_not_16_byte_aligned_or_not_contiguous(layout):
    """The streaming loop uses 16-byte loads from the first aligned element on and single loads around them; logits with
    a unit column stride but odd offsets or row strides, and logits with a non-unit column stride, take the other paths."""
    g = torch.Generator().manual_seed(21)
    rows, width, top_k = 5, 40000, 256
    if layout == "odd_offset":
        base = torch.randn(rows, width + 16, generator=g)
        view = lambda t: t[:, 3 : 3 + width]
    elif layout == "odd_row_stride":
        base = torch.randn(rows, width + 1, generator=g)
        view = lambda t: t[:, :width]
    else:
        base = torch.randn(width, rows, generator=g)
        view = lambda t: t.t()
    logits = view(base)
    starts = torch.tensor([0, 1, 2, 3, 17], dtype=torch.int32)
    ends = torch.tensor([width, width - 1, 30001, 9000, 18], dtype=torch.int32)
    want = torch.zeros(rows, top_k, dtype=torch.int32)
    c_oracle.top_k_per_row_prefill(logits, starts, ends, want, rows, logits.stride(0), logits.stride(1), top_k)
    dev = view(base.to(DEV))
    got = torch.full((rows, top_k), 7, dtype=torch.int32, device=DEV)
    flaggems_vllm.top_k_per_row_prefill(dev, starts.to(DEV), ends.to(DEV), got, rows, dev.stride(0), dev.stride(1), top_k)
    assert torch.equal(selected_values(logits, got, starts, ends, top_k), selected_values(logits, want, starts, ends, top_k))


@pytest.mark.gpu
def test_cluster_launch_replays_from_a_cuda_graph():
    """Decode steps run from CUDA graphs: the cluster launch (4 rows of 65536 -> 4 CTAs per row) must be capturable and a
    replay on new logits must select the new rows' values."""
    g = torch.Generator().manual_seed(9)
    logits = torch.randn(4, 65536, generator=g).to(DEV)
    seq = torch.tensor([65536, 40000, 9000, 300], dtype=torch.int32, device=DEV)
    idx = torch.zeros(4, 512, dtype=torch.int32, device=DEV)
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        flaggems_vllm.top_k_per_row_decode(logits, 1, seq, idx, 4, logits.stride(0), 1, 512)  # warm-up outside the capture
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=s):
            flaggems_vllm.top_k_per_row_decode(logits, 1, seq, idx, 4, logits.stride(0), 1, 512)
        fresh = torch.randn(4, 65536, generator=g)
        logits.copy_(fresh)
        idx.zero_()
        graph.replay()
    s.synchronize()
    want = torch.zeros(4, 512, dtype=torch.int32)
    c_oracle.top_k_per_row_decode(fresh, 1, seq.cpu(), want, 4, fresh.stride(0), 1, 512)
    ends = decode_ends(seq.cpu(), 1, 4)
    assert torch.equal(selected_values(fresh, idx, torch.zeros(4), ends, 512), selected_values(fresh, want, torch.zeros(4), ends, 512))


def test_host_checks_without_gpu():
    logits, idx = torch.zeros(2, 100), torch.zeros(2, 8, dtype=torch.int32)
    with pytest.raises(AssertionError, match="no CPU path"):
        flaggems_vllm.top_k_per_row_decode(logits, 1, torch.tensor([100, 100], dtype=torch.int32), idx, 2, 100, 1, 8)
    with pytest.raises(AssertionError):
        flaggems_vllm.top_k_per_row_prefill(logits, torch.zeros(2, dtype=torch.int32), torch.zeros(2, dtype=torch.int32), idx, 3, 100, 1, 8)
