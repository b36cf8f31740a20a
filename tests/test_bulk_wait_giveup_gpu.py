"""The give-up path of the bulk-copy kernel variant (csrc/prologue_bulk.cu), exercised without faulting anything.

Every wait of that kernel on a shared-memory barrier has a limit.  The self-test entry point makes ONE tile's loader
announce 16 bytes that it never sends, with a limit of about half a millisecond, so the waits on that tile's stage run
out.  What must then happen: the waiting roles give up, the CTA's other roles leave their loops, the loader lets the
copies it has already issued land, the kernel returns by itself, the device error word reads 1 and is cleared by the
read, every CTA that did not own the short tile has finished its work, and the next ordinary launch is as exact as ever.
Nothing here traps, reads a bad address or waits without a limit.
"""
from __future__ import annotations

import pytest
import torch

import flaggems_vllm
from flaggems_vllm import _native
from flaggems_vllm.testing import compare, workloads
from oracle import c_oracle

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
TILE = 16  # rows per tile of the shipped bulk shape


def test_wait_runs_out_kernel_returns_and_the_next_launch_is_exact():
    n, h, bs = 96, 64, 64  # 6 tiles of kv rows, then 384 tiles of q rows: a few tiles per CTA
    w = workloads.make("cpu_ref", device=DEV, seed=5, num_tokens=n, num_heads=h, num_blocks=8)
    q0, kc0 = w.q.clone(), w.k_cache.clone()
    q_ref, kc_ref = q0.cpu().clone(), kc0.cpu().clone()
    c_oracle.prologue(q_ref, w.kv.cpu(), kc_ref, w.slot_mapping.cpu(), w.position_ids.cpu(), w.cos_sin_cache.cpu(), w.eps, bs)

    kv_tiles = (n + TILE - 1) // TILE
    short_tile = kv_tiles + 11  # the 12th tile of q rows: q rows 176..191
    assert _native.device_error() == 0
    previous = _native.lib().dsv4_set_bulk_wait_cycles(1_000_000)
    try:
        stream = torch.cuda.current_stream().cuda_stream
        _native.check(_native.lib().dsv4_bulk_wait_selftest(
            w.q.data_ptr(), w.kv.data_ptr(), w.k_cache.data_ptr(), w.slot_mapping.data_ptr(), w.position_ids.data_ptr(),
            w.cos_sin_cache.data_ptr(), w.eps, n, h, n, bs, w.k_cache.stride(0), short_tile, stream))
        torch.cuda.synchronize()  # returns: the kernel ended by itself
    finally:
        assert _native.lib().dsv4_set_bulk_wait_cycles(previous) == 1_000_000
    assert _native.device_error() == 1, "the wait that ran out must be reported"
    assert _native.device_error() == 0, "reading the error word clears it"

    # the rows of the short tile were never processed; every tile of the other CTAs was, exactly
    rows = w.q.view(n * h, 512)
    rows0, rows_ref = q0.view(n * h, 512), q_ref.view(n * h, 512).to(DEV)
    lo = (short_tile - kv_tiles) * TILE
    assert torch.equal(rows[lo : lo + TILE], rows0[lo : lo + TILE]), "the short tile must be left as it was"
    done = (compare.bf16_ulp_distance(rows.cpu(), rows_ref.cpu()).amax(dim=1) <= 1)
    untouched = (rows == rows0).all(dim=1).cpu()
    assert bool((done | untouched).all()), "a row is neither finished nor untouched"
    total_tiles = kv_tiles + n * h // TILE
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    ctas = min(total_tiles, sms)
    # only tiles of the CTA that owned the short tile (same index modulo the grid) may be unfinished
    unfinished = torch.nonzero(~done).flatten() // TILE + kv_tiles
    assert unfinished.numel() >= TILE and bool(((unfinished - short_tile) % ctas == 0).all())
    assert bool((unfinished >= short_tile).all())
    assert torch.equal(w.k_cache.cpu(), kc_ref), "the kv tiles belong to other CTAs and must be complete"

    # an ordinary launch afterwards, both variants: exact, and no error reported
    for variant in (_native.VARIANT_BULK, _native.VARIANT_ROWS):
        w.q.copy_(q0), w.k_cache.copy_(kc0)
        prev = _native.set_variant(variant)
        try:
            flaggems_vllm.fused_deepseek_v4_qnorm_rope_kv_rope_quant_insert(*w.args())
            torch.cuda.synchronize()
        finally:
            _native.set_variant(prev)
        assert _native.device_error() == 0
        assert torch.equal(w.k_cache.cpu(), kc_ref)
        compare.assert_q_close(w.q.cpu(), q_ref)


def test_wait_limit_setter_round_trip():
    lib = _native.lib()
    default = lib.dsv4_set_bulk_wait_cycles(0)  # <= 0 only reads
    assert 0 < default <= 2_000_000_000
    assert lib.dsv4_set_bulk_wait_cycles(5_000_000_000) == default
    assert lib.dsv4_set_bulk_wait_cycles(default) == 2_000_000_000  # clamped
    assert lib.dsv4_set_bulk_wait_cycles(0) == default
