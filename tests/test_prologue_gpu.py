"""Parity of the CUDA prologue (called through the Python entry point -> C ABI) with the CPU
oracle and with the golden vectors of the upstream torch reference.

Bars (see flaggems_vllm.testing.compare): cache rows byte-identical (required: >= 99.9 % of e4m3
bytes identical, rest 1 ulp; scale bytes identical), untouched cache bytes bit-identical, q within
1 bf16 ulp.  Shape families follow the upstream tests
(tests/test_fused_deepseek_v4_qnorm_rope_kv_rope_quant_insert.py:358-573) and the five
benchmark configurations; the cases upstream does not cover (scattered slots, -1 among valid
slots, random positions, padded or unaligned block pitch, odd head counts) are added.
"""
from __future__ import annotations

import numpy as np
import pytest
import torch

import flaggems_vllm
from conftest import GOLDEN, SMALL_GOLDEN_CASES, load_golden
from flaggems_vllm import _native
from flaggems_vllm.testing import compare, workloads
from oracle import c_oracle

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
VARIANTS = {"rows": _native.VARIANT_ROWS, "bulk": _native.VARIANT_BULK}
op = flaggems_vllm.fused_deepseek_v4_qnorm_rope_kv_rope_quant_insert


@pytest.fixture(params=sorted(VARIANTS))
def variant(request):
    prev = _native.set_variant(VARIANTS[request.param])
    yield request.param
    _native.set_variant(prev)


@pytest.fixture(autouse=True)
def _free_device_memory():
    yield
    torch.cuda.empty_cache()


def oracle_of(q, kv, k_cache, slots, pos, cs, eps, bs):
    """Run the C oracle on host copies; returns (q_ref, k_cache_ref) on the host."""
    qh, kch = q.cpu().clone(), k_cache.cpu().clone()
    c_oracle.prologue(qh, kv.cpu(), kch, slots.cpu(), pos.cpu(), cs.cpu(), eps, bs)
    return qh, kch


def run_and_check(q, kv, k_cache, slots, pos, cs, eps, bs, *, q_ref=None, kc_ref=None):
    """Launch on the GPU, compare everything with the oracle (or the given expectations)."""
    if q_ref is None:
        q_ref, kc_ref = oracle_of(q, kv, k_cache, slots, pos, cs, eps, bs)
    kv_before, kc_before = kv.clone(), k_cache.clone()
    launches = _native.launch_count()
    op(q, kv, k_cache, slots, pos, cs, eps, bs)
    torch.cuda.synchronize()
    assert _native.launch_count() == launches + 1, "the operator is one kernel launch"
    assert _native.device_error() == 0, "a bounded wait inside the kernel ran out"
    assert torch.equal(kv, kv_before), "kv must not be written"
    compare.assert_untouched(k_cache, kc_before, slots, bs)
    kc_host = k_cache.cpu()
    assert torch.equal(kc_host, kc_ref), "cache differs from the oracle"
    compare.assert_cache_close(kc_host, kc_ref, slots.cpu(), bs, exact=True)
    return compare.assert_q_close(q.cpu(), q_ref)


def random_case(n, h, bs, nb, seed, *, n_insert=None, minus_one=0, stride_pad=0, zero_cache=False):
    g = torch.Generator().manual_seed(seed)
    q = torch.randn(n, h, 512, generator=g).to(torch.bfloat16)
    kv = torch.randn(n, 512, generator=g).to(torch.bfloat16)
    kc = torch.randint(0, 256, (nb, bs * 584 + stride_pad), generator=g, dtype=torch.uint8)
    if zero_cache:
        kc.zero_()
    n_ins = n if n_insert is None else n_insert
    slots = torch.randperm(nb * bs, generator=g)[:n_ins].to(torch.int64)
    if minus_one:
        slots[torch.randperm(n_ins, generator=g)[:minus_one]] = -1
    pos = torch.randint(0, 4096, (n,), generator=g, dtype=torch.int64)
    cs = workloads.cos_sin_table(4096)
    return [t.to(DEV) for t in (q, kv, kc, slots, pos, cs)]


# ---- golden vectors made by the upstream torch reference -------------------------------------


@pytest.mark.parametrize("case", SMALL_GOLDEN_CASES)
def test_golden_vectors(variant, case):
    g = load_golden(case)
    dev = {k: (v.to(DEV) if isinstance(v, torch.Tensor) else v) for k, v in g.items()}
    run_and_check(dev["q"], dev["kv"], dev["k_cache"], dev["slot_mapping"], dev["position_ids"], dev["cos_sin_cache"],
                  g["eps"], g["block_size"], q_ref=g["q_out"], kc_ref=g["k_cache_out"])


def test_cpu_ref_config_matches_upstream_golden(variant):
    """The benchmark configuration "CPU torch reference path, seed 0" (256 tokens x 8 heads)."""
    z = np.load(GOLDEN / "cpu_ref.npz")
    w = workloads.make("cpu_ref", device="cpu", seed=0)
    q, kv, kc, slots, pos, cs = [t.to(DEV) for t in (w.q, w.kv, w.k_cache, w.slot_mapping, w.position_ids, w.cos_sin_cache)]
    run_and_check(q, kv, kc, slots, pos, cs, w.eps, 64)
    d, s = compare.gather_rows(kc.cpu(), w.slot_mapping, 64)
    assert torch.equal(d, torch.from_numpy(z["rows_data"])) and torch.equal(s, torch.from_numpy(z["rows_scales"]))
    head = torch.from_numpy(z["q_out_head"].view(np.int16).copy()).view(torch.bfloat16)
    assert int(compare.bf16_ulp_distance(q[:48].cpu(), head).max()) <= 1


# ---- the upstream test families, against the oracle --------------------------------------------


@pytest.mark.parametrize("num_tokens", [1, 4, 17, 64])
@pytest.mark.parametrize("n_heads", [8, 64])
def test_q_path(variant, num_tokens, n_heads):
    """T:358-402: kv zero, every slot -1, positions 0..N-1; only q changes."""
    q, kv, kc, slots, pos, cs = random_case(num_tokens, n_heads, 16, 2, seed=0, zero_cache=True)
    kv.zero_(), slots.fill_(-1)
    pos.copy_(torch.arange(num_tokens))
    run_and_check(q, kv, kc, slots, pos, cs, 1e-6, 16)
    assert int(kc.abs().max()) == 0


@pytest.mark.parametrize("num_tokens", [1, 4, 17, 64])
@pytest.mark.parametrize("block_size", [16, 64])
def test_kv_path(variant, num_tokens, block_size):
    """T:419-462: one zero q head, kv random, slots 0..N-1."""
    nb = (num_tokens + block_size - 1) // block_size + 1
    q, kv, kc, slots, pos, cs = random_case(num_tokens, 1, block_size, nb, seed=1, zero_cache=True)
    q.zero_()
    slots.copy_(torch.arange(num_tokens)), pos.copy_(torch.arange(num_tokens))
    run_and_check(q, kv, kc, slots, pos, cs, 1e-6, block_size)


@pytest.mark.parametrize("num_tokens", [4, 17])
@pytest.mark.parametrize("pad", [1, 5])
@pytest.mark.parametrize("block_size", [16, 64])
def test_dp_padding(variant, num_tokens, pad, block_size):
    """T:468-515: slot_mapping shorter than q; padded tokens get q work, no cache write."""
    nb = (num_tokens + block_size - 1) // block_size + 1
    q, kv, kc, slots, pos, cs = random_case(num_tokens + pad, 2, block_size, nb, seed=3, n_insert=num_tokens)
    run_and_check(q, kv, kc, slots, pos, cs, 1e-6, block_size)


@pytest.mark.parametrize("num_tokens", [1, 4, 17, 64, 777])
@pytest.mark.parametrize("n_heads", [64, 128])
@pytest.mark.parametrize("block_size", [16, 64])
def test_combined(variant, num_tokens, n_heads, block_size):
    """T:521-573 (small sizes; the large ones are the configuration tests below)."""
    nb = (num_tokens + block_size - 1) // block_size + 1
    q, kv, kc, slots, pos, cs = random_case(num_tokens, n_heads, block_size, nb, seed=2)
    run_and_check(q, kv, kc, slots, pos, cs, 1e-6, block_size)


# ---- what upstream does not test ----------------------------------------------------------------


@pytest.mark.parametrize("n_heads", [1, 2, 3, 5, 7, 15, 17, 33, 100])
def test_head_counts_that_do_not_divide_the_row_tile(variant, n_heads):
    q, kv, kc, slots, pos, cs = random_case(53, n_heads, 16, 8, seed=10 + n_heads, minus_one=7)
    run_and_check(q, kv, kc, slots, pos, cs, 1e-6, 16)


def test_zero_heads_and_zero_tokens(variant):
    q, kv, kc, slots, pos, cs = random_case(9, 0, 16, 2, seed=4)
    run_and_check(q, kv, kc, slots, pos, cs, 1e-6, 16)
    before = kc.clone()
    e = torch.empty
    op(e(0, 8, 512, dtype=torch.bfloat16, device=DEV), e(0, 512, dtype=torch.bfloat16, device=DEV), kc,
       e(0, dtype=torch.int64, device=DEV), e(0, dtype=torch.int64, device=DEV), cs, 1e-6, 16)
    torch.cuda.synchronize()
    assert torch.equal(kc, before)


@pytest.mark.parametrize("stride_pad,offset", [(64, 0), (16, 16), (8, 0), (1, 0), (0, 8), (0, 3)])
def test_block_pitch_and_alignment(variant, stride_pad, offset):
    """Padded block pitch and cache bases that are not 16-byte aligned (byte-store path)."""
    bs, nb, n = 16, 5, 40
    q, kv, kc, slots, pos, cs = random_case(n, 4, bs, nb, seed=20 + stride_pad + offset, minus_one=3, stride_pad=stride_pad)
    pitch = kc.shape[1]
    backing = torch.randint(0, 256, (nb * pitch + 64,), dtype=torch.uint8, device=DEV)
    view = backing[offset : offset + nb * pitch].view(nb, pitch)
    view.copy_(kc)
    guard = backing.clone()
    run_and_check(q, kv, view, slots, pos, cs, 1e-6, bs)
    assert torch.equal(backing[:offset], guard[:offset]) and torch.equal(backing[offset + nb * pitch :], guard[offset + nb * pitch :])


def test_guard_bands_around_q_kv_and_cache(variant):
    """Inputs carved out of larger sentinel-filled buffers: nothing outside them is written."""
    n, h, bs, nb = 37, 6, 16, 4
    q, kv, kc, slots, pos, cs = random_case(n, h, bs, nb, seed=30, minus_one=5)
    band = 4096

    def carve(t):
        raw = torch.full((t.numel() * t.element_size() + 2 * band,), 0xA5, dtype=torch.uint8, device=DEV)
        inner = raw[band : band + t.numel() * t.element_size()].view(t.dtype).view(t.shape)
        inner.copy_(t)
        return raw, inner

    raw_q, q2 = carve(q)
    raw_kv, kv2 = carve(kv)
    raw_kc, kc2 = carve(kc)
    run_and_check(q2, kv2, kc2, slots, pos, cs, 1e-6, bs)
    for raw in (raw_q, raw_kv, raw_kc):
        assert int((raw[:band] != 0xA5).sum()) == 0 and int((raw[-band:] != 0xA5).sum()) == 0


def test_checked_build_reports_and_skips_bad_indices():
    """The range-checked entry point stands in for a memory checker: out-of-range positions and
    slots are skipped and reported, everything else is processed as usual."""
    n, h, bs, nb = 64, 4, 16, 6
    q, kv, kc, slots, pos, cs = random_case(n, h, bs, nb, seed=40)
    checked = flaggems_vllm.fused_deepseek_v4_qnorm_rope_kv_rope_quant_insert_checked
    q0, kc0 = q.clone(), kc.clone()
    assert checked(q, kv, kc, slots, pos, cs, 1e-6, bs) == 0
    q_ref, kc_ref = oracle_of(q0, kv, kc0, slots, pos, cs, 1e-6, bs)
    assert torch.equal(kc.cpu(), kc_ref)
    compare.assert_q_close(q.cpu(), q_ref)

    q, kc = q0.clone(), kc0.clone()
    bad_pos, bad_slot = [3, 17], [5, 40]
    pos2, slots2 = pos.clone(), slots.clone()
    pos2[bad_pos[0]], pos2[bad_pos[1]] = 4096, -1
    slots2[bad_slot[0]], slots2[bad_slot[1]] = nb * bs, nb * bs + 1000
    assert checked(q, kv, kc, slots2, pos2, cs, 1e-6, bs) == 3
    # expectation: bad-position tokens untouched everywhere; bad-slot tokens only lose the insert
    pos_ok, slots_exp = pos2.clone(), slots2.clone()
    pos_ok[bad_pos] = 0
    slots_exp[bad_pos + bad_slot] = -1
    q_ref, kc_ref = oracle_of(q0, kv, kc0, slots_exp, pos_ok, cs, 1e-6, bs)
    q_ref[bad_pos] = q0[bad_pos].cpu()
    assert torch.equal(kc.cpu(), kc_ref)
    compare.assert_q_close(q.cpu(), q_ref)


def test_stream_and_cuda_graph_capture(variant):
    """Runs on the caller's current stream and can be captured: no allocation, no sync inside."""
    q, kv, kc, slots, pos, cs = random_case(33, 16, 16, 4, seed=50)
    q_ref, kc_ref = oracle_of(q, kv, kc, slots, pos, cs, 1e-6, 16)
    q_in = q.clone()
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        op(q, kv, kc, slots, pos, cs, 1e-6, 16)  # warm-up outside capture
        q.copy_(q_in)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=s):
            op(q, kv, kc, slots, pos, cs, 1e-6, 16)
        q.copy_(q_in)
        graph.replay()
    s.synchronize()
    assert torch.equal(kc.cpu(), kc_ref)
    compare.assert_q_close(q.cpu(), q_ref)


# ---- the benchmark configurations ---------------------------------------------------------------


def test_decode_config(variant):
    w = workloads.make("decode", device=DEV, seed=0)
    run_and_check(*w.args())


def test_prefill_config_full_comparison(variant):
    """8192 tokens x 128 heads, compared in full with the oracle (q is 1 GiB)."""
    w = workloads.make("prefill", device=DEV, seed=0)
    q_ref, _ = oracle_of(w.q, w.kv, torch.zeros(1, 64 * 584, dtype=torch.uint8), w.slot_mapping[:0], w.position_ids,
                         w.cos_sin_cache, w.eps, 64)
    check_cache_rows_against_compact_oracle(w, run=True)
    st = compare.assert_q_close(w.q.cpu(), q_ref)
    assert st["elements"] == 8192 * 128 * 512


def check_cache_rows_against_compact_oracle(w, run: bool):
    """Large caches are not copied to the host: the oracle inserts the same tokens into a compact
    cache (slot = rank among the valid slots; a row's bytes do not depend on where it is stored) and
    the rows are compared; untouched bytes are checked on the device."""
    bs = w.cache_block_size
    before = w.k_cache.clone()
    kv_before = w.kv.clone()
    if run:
        op(*w.args())
        torch.cuda.synchronize()
    assert torch.equal(w.kv, kv_before)
    compare.assert_untouched(w.k_cache, before, w.slot_mapping, bs)
    del before
    slots = w.slot_mapping.cpu()
    valid = slots >= 0
    compact = torch.full_like(slots, -1)
    compact[valid] = torch.arange(int(valid.sum()))
    small = torch.zeros((int(valid.sum()) + bs - 1) // bs + 1, bs * 584, dtype=torch.uint8)
    n_ins = slots.shape[0]
    c_oracle.prologue(torch.empty(n_ins, 0, 512, dtype=torch.bfloat16), w.kv[:n_ins].cpu(), small, compact,
                      w.position_ids[:n_ins].cpu(), w.cos_sin_cache.cpu(), w.eps, bs)
    d_ref, s_ref = compare.gather_rows(small, compact[valid], bs)
    d, s = compare.gather_rows(w.k_cache, w.slot_mapping[w.slot_mapping >= 0], bs)
    assert torch.equal(d.cpu(), d_ref), "cached data rows differ from the oracle"
    assert torch.equal(s.cpu(), s_ref), "cached scale rows differ from the oracle"


def test_long_prefill_config_sampled(variant):
    """32768 tokens x 128 heads, 10 % slots -1, 1 % outlier rows (q is 4 GiB): every cache row and
    every untouched byte is checked; q is checked on all outlier tokens plus a random sample."""
    w = workloads.make("long_prefill", device=DEV, seed=0)
    g = torch.Generator().manual_seed(123)
    outliers = torch.nonzero(w.kv.float().abs().amax(dim=1) > 20.0).flatten().cpu()
    sample = torch.unique(torch.cat([outliers, torch.randperm(w.num_tokens, generator=g)[:512],
                                     torch.tensor([0, w.num_tokens - 1])]))
    q_in = w.q[sample.to(DEV)].cpu()
    check_cache_rows_against_compact_oracle(w, run=True)
    pos = w.position_ids.cpu()[sample]
    c_oracle.prologue(q_in, torch.empty(sample.numel(), 512, dtype=torch.bfloat16), torch.zeros(1, 64 * 584, dtype=torch.uint8),
                      torch.empty(0, dtype=torch.int64), pos, w.cos_sin_cache.cpu(), w.eps, 64)
    st = compare.assert_q_close(w.q[sample.to(DEV)].cpu(), q_in)
    assert outliers.numel() >= 300 and st["elements"] == sample.numel() * 128 * 512
    # size-independent property on the whole tensor: every normalised row has unit RMS
    for a in range(0, w.num_tokens, 4096):
        rms = w.q[a : a + 4096, :, :].float().pow(2).mean(dim=-1).sqrt()
        assert float((rms - 1.0).abs().max()) < 5e-3


def test_sharded_config_ranks_are_independent(variant):
    """Two shards of the token-sharded configuration at reduced size: each rank's result equals the
    oracle on that rank's tokens alone (no cross-rank state), on caches of their own."""
    for rank in range(2):
        w = workloads.make("sharded", device=DEV, seed=0, rank=rank, world=2, total_tokens=8192 + 4096,
                           num_heads=16, num_blocks=1024)
        run_and_check(*w.args())


def test_full_size_properties_determinism_and_slot_invariance(variant):
    """At the prefill size: two runs from the same inputs give identical bytes, and the bytes of a
    cached row do not depend on the slot it is stored in."""
    w = workloads.make("prefill", device=DEV, seed=1)
    q0, kc0 = w.q.clone(), w.k_cache.clone()
    op(*w.args())
    q1, kc1 = w.q.clone(), w.k_cache.clone()
    w.q.copy_(q0), w.k_cache.copy_(kc0)
    op(*w.args())
    torch.cuda.synchronize()
    assert torch.equal(w.q.view(torch.int16), q1.view(torch.int16)) and torch.equal(w.k_cache, kc1)
    del q1, kc1
    other = torch.randperm(w.k_cache.shape[0] * 64, device=DEV)[: w.num_tokens].to(torch.int64)
    d1, s1 = compare.gather_rows(w.k_cache, w.slot_mapping, 64)
    d1, s1 = d1.clone(), s1.clone()
    w.q.copy_(q0), w.k_cache.copy_(kc0)
    op(w.q, w.kv, w.k_cache, other, w.position_ids, w.cos_sin_cache, w.eps, 64)
    d2, s2 = compare.gather_rows(w.k_cache, other, 64)
    assert torch.equal(d1, d2) and torch.equal(s1, s2)


def test_hbm_probe_modes_leave_or_fill_the_buffer():
    """The ceiling probe: in-place and read-only modes leave the buffer unchanged, write-only fills
    every byte of the requested rows and nothing after them."""
    rows = 1000
    buf = torch.randint(0, 256, ((rows + 8) * 1024,), dtype=torch.uint8, device=DEV)
    before = buf.clone()
    from flaggems_vllm.testing import hbm_probe

    stream = torch.cuda.current_stream().cuda_stream
    for mode in (0, 1):
        hbm_probe.probe(mode, buf.data_ptr(), rows, stream)
        torch.cuda.synchronize()
        assert torch.equal(buf, before)
    hbm_probe.probe(2, buf.data_ptr(), rows, stream)
    torch.cuda.synchronize()
    assert torch.equal(buf[rows * 1024 :], before[rows * 1024 :])
    assert not torch.equal(buf[: rows * 1024], before[: rows * 1024])


@pytest.mark.parametrize("n_heads,padded", [(8, 16), (7, 8), (64, 64), (128, 192), (1, 3)])
def test_out_of_place_padded_form(n_heads, padded):
    """The nine-argument form: q untouched, result in a new [N, padded, 512] tensor with zero padding heads,
    cache identical to the in-place operator's."""
    q, kv, kc, slots, pos, cs = random_case(45, n_heads, 16, 6, seed=60 + n_heads, minus_one=4)
    q_ref, kc_ref = oracle_of(q, kv, kc, slots, pos, cs, 1e-6, 16)
    q_before = q.clone()
    launches = _native.launch_count()
    out = flaggems_vllm.fused_deepseek_v4_qnorm_rope_kv_rope_quant_insert_padded(q, kv, kc, slots, pos, cs, padded, 1e-6, 16)
    torch.cuda.synchronize()
    assert _native.launch_count() == launches + 1
    assert torch.equal(q, q_before), "q is read-only in this form"
    assert out.shape == (45, padded, 512)
    compare.assert_q_close(out[:, :n_heads].cpu().contiguous(), q_ref)
    assert int((out[:, n_heads:].view(torch.int16) != 0).sum()) == 0, "padding heads must be zero"
    assert torch.equal(kc.cpu(), kc_ref)
    # identical bits to the in-place operator
    op(q, kv, kc, slots, pos, cs, 1e-6, 16)
    assert torch.equal(out[:, :n_heads].contiguous().view(torch.int16), q.view(torch.int16))


@pytest.mark.parametrize("num_tokens,n_heads", [(131072, 128)])
def test_largest_upstream_size_sampled(variant, num_tokens, n_heads):
    """The largest size of the upstream combined test (T:531: 131072 tokens x 128 heads, q = 16 GiB, byte offsets
    beyond 2^32, positions up to 131071, arange slots): tokens sampled from the start, the 4 GiB boundaries and the
    end are compared with the oracle; every cache row is compared."""
    g = torch.Generator(device=DEV).manual_seed(2)
    q = torch.empty(num_tokens, n_heads, 512, dtype=torch.bfloat16, device=DEV)
    for a in range(0, num_tokens, 8192):
        q[a : a + 8192].copy_(torch.randn(8192, n_heads, 512, generator=g, device=DEV))
    kv = torch.randn(num_tokens, 512, generator=g, device=DEV).to(torch.bfloat16)
    bs = 64
    k_cache = torch.zeros(num_tokens // bs + 1, bs * 584, dtype=torch.uint8, device=DEV)
    pos = torch.arange(num_tokens, dtype=torch.int64, device=DEV)
    slots = torch.arange(num_tokens, dtype=torch.int64, device=DEV)
    cs = workloads.cos_sin_table(num_tokens, theta=100000.0, device=DEV)
    per_4gib = (1 << 32) // (n_heads * 1024)
    sample = torch.unique(torch.cat([torch.arange(0, 8), torch.arange(num_tokens - 8, num_tokens)] +
                                    [torch.arange(k * per_4gib - 4, k * per_4gib + 4) for k in range(1, num_tokens // per_4gib)] +
                                    [torch.randint(0, num_tokens, (256,))]))
    q_in = q[sample.to(DEV)].cpu()
    w = workloads.Workload("largest", q, kv, k_cache, slots, pos, cs, 1e-6, bs)
    check_cache_rows_against_compact_oracle(w, run=True)
    assert _native.device_error() == 0
    c_oracle.prologue(q_in, torch.empty(sample.numel(), 512, dtype=torch.bfloat16), torch.zeros(1, bs * 584, dtype=torch.uint8),
                      torch.empty(0, dtype=torch.int64), sample.clone(), cs.cpu(), 1e-6, bs)
    compare.assert_q_close(q[sample.to(DEV)].cpu(), q_in)
    # every row of the 16 GiB tensor was normalised: unit RMS everywhere
    for a in range(0, num_tokens, 8192):
        rms = q[a : a + 8192].float().pow(2).mean(dim=-1).sqrt()
        assert float((rms - 1.0).abs().max()) < 5e-3


def _vllm_kernel():
    """vLLM's own CUDA kernel for this operator, if the installed wheel has it (nine-argument form, returns the
    padded q); None otherwise.  A library kernel used only as a cross-check, as the upstream test does (T:629-681)."""
    try:
        import vllm._custom_ops  # noqa: F401 - registers torch.ops._C

        return torch.ops._C.fused_deepseek_v4_qnorm_rope_kv_rope_quant_insert
    except Exception:
        return None


@pytest.mark.parametrize("num_tokens", [17, 512, 777, 4096])
@pytest.mark.parametrize("n_heads", [64, 128])
@pytest.mark.parametrize("block_size", [16, 64])
def test_matches_vllm_kernel_if_present(num_tokens, n_heads, block_size):
    """Cross-check against vLLM's kernel (shapes of T:629-640): e4m3 bytes and scale bytes identical, q and the
    cached RoPE values within 1 bf16 ulp (that kernel contracts the rotation into FMAs)."""
    kernel = _vllm_kernel()
    if kernel is None:
        pytest.skip("vLLM's _C operator is not available")
    nb = (num_tokens + block_size - 1) // block_size + 1
    q, kv, kc, slots, pos, cs = random_case(num_tokens, n_heads, block_size, nb, seed=4, zero_cache=True)
    kc_ref = kc.clone()
    try:
        q_ref = kernel(q.clone(), kv, kc_ref, slots, pos, cs, n_heads, 1e-6, block_size)
        torch.cuda.synchronize()
    except Exception as e:  # another signature in another vLLM release
        pytest.skip("vLLM kernel present but not callable with nine arguments: " + str(e).splitlines()[0])
    op(q, kv, kc, slots, pos, cs, 1e-6, block_size)
    torch.cuda.synchronize()
    compare.assert_q_close(q.cpu(), q_ref.cpu())
    compare.assert_untouched(kc, kc_ref, slots, block_size)
    st = compare.assert_cache_close(kc.cpu(), kc_ref.cpu(), slots.cpu(), block_size, exact=False)
    assert st["fp8_identical_fraction"] == 1.0 and st["scale_bytes_equal"]


@pytest.mark.parametrize("seed", range(24))
def test_random_shapes(variant, seed):
    """Seeded random geometry: token and head counts, block size (1..128, not only powers of two), block pitch,
    slot_mapping length, share of -1 slots."""
    g = torch.Generator().manual_seed(1000 + seed)
    r = lambda lo, hi: int(torch.randint(lo, hi + 1, (1,), generator=g))  # noqa: E731
    n, h = r(1, 300), r(0, 40)
    bs = [1, 2, 3, 16, 24, 64, 128][r(0, 6)]
    nb = (n + bs - 1) // bs + r(1, 3)
    n_ins = r(0, n)
    pad = [0, 0, 16, 8, 1][r(0, 4)]
    q, kv, kc, slots, pos, cs = random_case(n, h, bs, nb, seed=2000 + seed, n_insert=n_ins, minus_one=n_ins // 5, stride_pad=pad)
    run_and_check(q, kv, kc, slots, pos, cs, 1e-6 if seed % 2 else 1e-5, bs)


def test_direct_c_abi_calls():
    """Straight through ctypes, without the Python wrapper: the legacy default stream (NULL), rejection of a q
    pointer on an odd address (nothing launched), and a zero-token call."""
    q, kv, kc, slots, pos, cs = random_case(21, 4, 16, 3, seed=70)
    q_ref, kc_ref = oracle_of(q, kv, kc, slots, pos, cs, 1e-6, 16)
    lib = _native.lib()
    args = lambda qp: (qp, kv.data_ptr(), kc.data_ptr(), slots.data_ptr(), pos.data_ptr(), cs.data_ptr(), 1e-6, 21, 4, 21, 16,  # noqa: E731
                       kc.stride(0), None)
    before = _native.launch_count()
    assert lib.dsv4_qnorm_rope_kv_insert(*args(q.data_ptr() + 1)) == -3
    assert lib.dsv4_qnorm_rope_kv_insert(q.data_ptr(), kv.data_ptr(), kc.data_ptr(), slots.data_ptr(), pos.data_ptr(), cs.data_ptr(),
                                         1e-6, 0, 4, 0, 16, kc.stride(0), None) == 0
    assert _native.launch_count() == before
    torch.cuda.synchronize()
    assert lib.dsv4_qnorm_rope_kv_insert(*args(q.data_ptr())) == 0
    torch.cuda.synchronize()
    assert _native.launch_count() == before + 1
    assert torch.equal(kc.cpu(), kc_ref)
    compare.assert_q_close(q.cpu(), q_ref)
    assert lib.dsv4_error_string(-3).decode()


def test_kernel_reproduces_the_upstream_flash_mla_cache_builder():
    """Same independent upstream statement of the cache format (see tests/test_oracle_golden.py), both kernel variants."""
    z = np.load(GOLDEN / "flash_mla_builder_cache.npz")
    kv = torch.from_numpy(z["kv"].view(np.int16).copy()).view(torch.bfloat16).to("cuda:0")
    want, bs, n = torch.from_numpy(z["cache"].copy()), int(z["block_size"]), kv.shape[0]
    table = torch.cat([torch.ones(2, 32), torch.zeros(2, 32)], dim=1).contiguous().to("cuda:0")
    for variant in (1, 2):
        previous = _native.set_variant(variant)
        try:
            cache = torch.zeros_like(want).to("cuda:0")
            flaggems_vllm.fused_deepseek_v4_qnorm_rope_kv_rope_quant_insert(
                torch.ones(n, 1, 512, dtype=torch.bfloat16, device="cuda:0"), kv, cache, torch.arange(n, device="cuda:0"),
                torch.zeros(n, dtype=torch.int64, device="cuda:0"), table, 1e-6, bs)
            assert torch.equal(cache.cpu(), want)
        finally:
            _native.set_variant(previous)


@pytest.mark.parametrize("mode", [1, 2])
def test_programmatic_dependent_launch_gives_the_same_result(mode):
    """In launch modes 1 and 2 (dsv4_set_pdl) the kernel may start before the kernel in front of it has finished.  Mode 2,
    the default, reads nothing before that kernel is done: every input, positions and slots included, may come from the
    kernel right in front.  Mode 1 waits only before touching q / kv / cache.  A producer directly in front of the
    prologue, eager and replayed from a CUDA graph, must give the bytes of a plain launch (mode 0)."""
    q0, kv0, kc0, slots0, pos0, cs = random_case(300, 16, 64, 12, seed=77)
    want_q, want_kv, want_kc = q0.clone(), kv0.clone(), kc0.clone()
    previous = _native.set_pdl(0)
    try:
        op(want_q, want_kv, want_kc, slots0, pos0, cs, 1e-6, 64)
        q_ref, kc_ref = oracle_of(q0, kv0, kc0, slots0, pos0, cs, 1e-6, 64)
        assert torch.equal(want_kc.cpu(), kc_ref)
        assert _native.set_pdl(mode) == 0
        q, kv, kc = torch.empty_like(q0), torch.empty_like(kv0), kc0.clone()
        slots, pos = (torch.zeros_like(slots0), torch.zeros_like(pos0)) if mode == 2 else (slots0, pos0)

        def produce_then_consume():
            q.copy_(q0)  # the producers of the inputs are the kernels right in front of the prologue
            kv.copy_(kv0)
            if mode == 2:
                slots.copy_(slots0)
                pos.copy_(pos0)
            op(q, kv, kc, slots, pos, cs, 1e-6, 64)
            if mode == 2:  # and the kernel behind it may overwrite them at once
                slots.zero_()
                pos.zero_()

        produce_then_consume()
        torch.cuda.synchronize()
        assert torch.equal(q, want_q) and torch.equal(kc, want_kc)
        s = torch.cuda.Stream()
        s.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(s):
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=s):
                produce_then_consume()
                produce_then_consume()
            q.zero_(), kc.copy_(kc0)
            graph.replay()
        s.synchronize()
        assert torch.equal(q, want_q) and torch.equal(kc, want_kc)
    finally:
        _native.set_pdl(previous)
    assert _native.set_pdl(previous) == previous


@pytest.mark.parametrize("staging", [0, 1])
@pytest.mark.parametrize("pdl", [0, 1, 2])
@pytest.mark.parametrize("n,h", [(37, 9), (600, 128)])
def test_every_launch_mode_and_table_staging_gives_the_oracle_result(staging, pdl, n, h):
    """The rows kernel has two ways to fetch the cos/sin rows (per warp into registers, or once per CTA through shared
    memory; chosen by launch size unless forced) and three launch modes; the result does not depend on either.  Both
    sizes are run in both staging modes: a launch of a few CTAs and one above the size at which the library switches."""
    q, kv, kc, slots, pos, cs = random_case(n, h, 64, n // 64 + 3, seed=1000 + n, minus_one=max(1, n // 10))
    previous_staging, previous_pdl = _native.set_table_staging(staging), _native.set_pdl(pdl)
    try:
        run_and_check(q, kv, kc, slots, pos, cs, 1e-6, 64)
    finally:
        _native.set_table_staging(previous_staging)
        _native.set_pdl(previous_pdl)
    assert _native.set_table_staging(previous_staging) == previous_staging


@pytest.mark.parametrize("q_off,kv_off,cs_off", [(1, 0, 0), (0, 3, 0), (0, 0, 1), (5, 7, 3), (4, 4, 2)])
@pytest.mark.parametrize("n,h,bs", [(1, 1, 16), (19, 8, 64), (70, 33, 16)])
def test_contiguous_views_that_do_not_start_on_16_bytes(variant, q_off, kv_off, cs_off, n, h, bs):
    """The reference asks for contiguous tensors only (:320 there); a contiguous view may start any number of elements
    into its storage (a slice of a fused projection's output).  q, kv and the table offset by q_off / kv_off / cs_off
    elements: such calls take the any-alignment kernel, under either variant, and meet the same bars."""
    q, kv, kc, slots, pos, cs = random_case(n, h, bs, n // bs + 2, seed=31 * n + q_off + kv_off, minus_one=n // 5)

    def shifted(t, off):
        flat = torch.empty(t.numel() + off, dtype=t.dtype, device=t.device)
        view = flat[off:].view(t.shape)
        view.copy_(t)
        return view

    q2, kv2, cs2 = shifted(q, q_off), shifted(kv, kv_off), shifted(cs, cs_off)
    assert q2.is_contiguous() and kv2.is_contiguous() and cs2.is_contiguous()
    assert any(t.data_ptr() % 16 for t in (q2, kv2, cs2))
    run_and_check(q2, kv2, kc, slots, pos, cs2, 1e-6, bs)


@pytest.mark.parametrize("mode", [0, 1, 2])
def test_graph_capture_with_a_cross_stream_join_in_front(mode):
    """The operator captured right behind a join of two streams (kv produced on a side stream, q on the capturing one):
    in the dependent-launch modes the launch carries the programmatic-serialization attribute, which must degrade to an
    ordinary dependency where the node in front is not a kernel of the same stream.  Replayed twice, exact both times."""
    q0, kv0, kc0, slots, pos, cs = random_case(150, 12, 64, 6, seed=91)
    q_ref, kc_ref = oracle_of(q0, kv0, kc0, slots, pos, cs, 1e-6, 64)
    q, kv, kc = torch.zeros_like(q0), torch.zeros_like(kv0), kc0.clone()
    previous = _native.set_pdl(mode)
    try:
        main, side = torch.cuda.Stream(), torch.cuda.Stream()
        main.wait_stream(torch.cuda.current_stream())
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.stream(main):
            op(q0.clone(), kv0, kc0.clone(), slots, pos, cs, 1e-6, 64)  # warm-up outside the capture
            main.synchronize()
            with torch.cuda.graph(graph, stream=main):
                side.wait_stream(main)
                with torch.cuda.stream(side):
                    kv.copy_(kv0)
                q.copy_(q0)
                main.wait_stream(side)
                op(q, kv, kc, slots, pos, cs, 1e-6, 64)
        for _ in range(2):
            q.zero_(), kv.zero_(), kc.copy_(kc0)
            torch.cuda.synchronize()
            graph.replay()
            torch.cuda.synchronize()
            assert torch.equal(kc.cpu(), kc_ref)
            compare.assert_q_close(q.cpu(), q_ref)
    finally:
        _native.set_pdl(previous)
    assert _native.device_error() == 0
