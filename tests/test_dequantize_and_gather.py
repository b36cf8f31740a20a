"""`dequantize_and_gather_k_cache` (request / block-table form): oracle vs the upstream test's
known-answer vectors on CPU; CUDA kernel vs the same vectors and vs the oracle on random caches."""
from __future__ import annotations

import numpy as np
import pytest
import torch

import flaggems_vllm
from conftest import GOLDEN, _bf16
from oracle import c_oracle

GATHER_GOLDEN = sorted(p.stem for p in GOLDEN.glob("gather_*.npz"))
DEV = "cuda:0"


def load(name):
    z = np.load(GOLDEN / f"{name}.npz")
    t = {k: torch.from_numpy(z[k].copy()) for k in ("k_cache", "seq_lens", "gather_lens", "block_table")}
    t["expected"] = _bf16(z["expected"])
    t.update({k: int(z[k]) for k in ("block_size", "nope_dim", "rope_dim", "scale_slots")})
    return t


def test_golden_files_exist():
    assert len(GATHER_GOLDEN) >= 3


@pytest.mark.parametrize("name", GATHER_GOLDEN)
def test_oracle_reproduces_upstream_known_answers(name):
    g = load(name)
    out = torch.full_like(g["expected"], 7.0)
    c_oracle.dequantize_and_gather(out, g["k_cache"], g["seq_lens"], g["gather_lens"], g["block_table"], g["block_size"],
                                   rope_dim=g["rope_dim"], nope_dim=g["nope_dim"], scale_slots=g["scale_slots"])
    assert torch.equal(out.view(torch.int16), g["expected"].view(torch.int16))


@pytest.mark.gpu
@pytest.mark.parametrize("index_dtype", [torch.int32, torch.int64])
@pytest.mark.parametrize("name", GATHER_GOLDEN)
def test_kernel_reproduces_upstream_known_answers(name, index_dtype):
    g = load(name)
    out = torch.full(g["expected"].shape, 7.0, dtype=torch.bfloat16, device=DEV)
    flaggems_vllm.dequantize_and_gather_k_cache(
        out, g["k_cache"].to(DEV), g["seq_lens"].to(DEV, index_dtype), g["gather_lens"].to(DEV, index_dtype),
        g["block_table"].to(DEV, index_dtype), g["block_size"], rope_dim=g["rope_dim"], nope_dim=g["nope_dim"],
        scale_slots=g["scale_slots"])
    assert torch.equal(out.cpu().view(torch.int16), g["expected"].view(torch.int16))


def random_case(seed, batch, max_seq, bs, nope, rope, with_gather=True, extra_out=0, offset=0, pad=0):
    g = torch.Generator().manual_seed(seed)
    slots = (nope + 63) // 64 + (1 if nope % 64 == 0 else 0)
    seq = torch.randint(1, max_seq + 1, (batch,), generator=g, dtype=torch.int32)
    gather = (torch.rand(batch, generator=g) * seq).ceil().to(torch.int32).clamp(min=1) if with_gather else None
    bps = (max_seq + bs - 1) // bs
    nb = batch * bps + 3
    table = torch.randperm(nb, generator=g)[: batch * bps].to(torch.int32).view(batch, bps)
    kc = torch.randint(0, 256, (nb, bs * (nope + 2 * rope + slots) + pad), generator=g, dtype=torch.uint8)
    kc[(kc & 0x7F) == 0x7F] = 0x41  # no e4m3 NaN codes: NaN payloads are not comparable bit for bit
    region = kc[:, bs * (nope + 2 * rope) : bs * (nope + 2 * rope + slots)]
    region.copy_(torch.randint(100, 140, region.shape, generator=g, dtype=torch.uint8))
    t_out = int((gather if with_gather else seq).max()) + offset + extra_out
    return seq, gather, table, kc, slots, t_out


@pytest.mark.gpu
@pytest.mark.parametrize("batch,max_seq,bs,nope,rope,with_gather,offset,pad", [
    (4, 300, 64, 448, 64, True, 0, 0), (5, 1000, 64, 448, 64, False, 0, 0), (3, 200, 16, 448, 64, True, 5, 0),
    (2, 90, 64, 448, 64, True, 0, 8), (3, 77, 4, 64, 16, True, 2, 0), (2, 50, 8, 100, 32, True, 0, 0),
    (70, 40, 64, 448, 64, True, 0, 0), (4, 200, 24, 448, 64, True, 0, 0),  # 24: a block size that is not a power of two
])
def test_kernel_matches_oracle_on_random_caches(batch, max_seq, bs, nope, rope, with_gather, offset, pad):
    seq, gather, table, kc, slots, t_out = random_case(batch * 7 + max_seq, batch, max_seq, bs, nope, rope, with_gather,
                                                       extra_out=2, offset=offset, pad=pad)
    want = torch.full((batch + 1, t_out, nope + rope), 3.0, dtype=torch.bfloat16)
    c_oracle.dequantize_and_gather(want, kc, seq, gather, table, bs, offset=offset, rope_dim=rope, nope_dim=nope,
                                   scale_slots=slots)
    out = torch.full(want.shape, 3.0, dtype=torch.bfloat16, device=DEV)
    flaggems_vllm.dequantize_and_gather_k_cache(out, kc.to(DEV), seq.to(DEV), None if gather is None else gather.to(DEV),
                                                table.to(DEV), bs, offset, rope, nope, slots)
    assert torch.equal(out.cpu().view(torch.int16), want.view(torch.int16)), "incl. rows the call must not touch"


@pytest.mark.gpu
def test_strided_output_and_3d_cache():
    """out as a slice of a wider buffer (rows not 16-byte aligned -> scalar path) and a [blocks, bs, 584] cache."""
    seq, gather, table, kc, slots, t_out = random_case(99, 3, 120, 64, 448, 64)
    want = torch.zeros(3, t_out, 512, dtype=torch.bfloat16)
    c_oracle.dequantize_and_gather(want, kc, seq, gather, table, 64)
    wide = torch.zeros(3, t_out, 512 + 6, dtype=torch.bfloat16, device=DEV)
    out = wide[:, :, 3 : 3 + 512]
    flaggems_vllm.dequantize_and_gather_k_cache(out, kc.view(-1, 64, 584).to(DEV), seq.to(DEV), gather.to(DEV),
                                                table.to(DEV), 64)
    assert torch.equal(out.cpu().contiguous().view(torch.int16), want.view(torch.int16))
    assert int(wide[:, :, :3].abs().max()) == 0 and int(wide[:, :, 515:].abs().max()) == 0


@pytest.mark.gpu
def test_prologue_then_reader_round_trip_through_block_table():
    """Tokens inserted by the prologue at slots derived from a block table come back through the same
    table: RoPE part bit-identical to the oracle's cache, de-quantised part equal to the oracle reader."""
    from flaggems_vllm.testing import workloads

    w = workloads.make("prefill", device=DEV, seed=3, num_heads=1, num_tokens=4096, num_blocks=256)
    flaggems_vllm.fused_deepseek_v4_qnorm_rope_kv_rope_quant_insert(*w.args())
    # the prefill workload fills whole blocks in token order: 2 requests of 2048 tokens = 32 blocks each
    table = (w.slot_mapping[::64] // 64).to(torch.int32).view(2, 32).contiguous()
    seq = torch.tensor([2048, 2048], dtype=torch.int32, device=DEV)
    out = torch.empty(2, 2048, 512, dtype=torch.bfloat16, device=DEV)
    flaggems_vllm.dequantize_and_gather_k_cache(out, w.k_cache, seq, None, table, 64)
    rows = flaggems_vllm.gather_dequant_k_cache_slots(w.k_cache, w.slot_mapping, 64)
    assert torch.equal(out.view(-1, 512).view(torch.int16), rows.view(torch.int16))
    want = torch.empty(2, 2048, 512, dtype=torch.bfloat16)
    c_oracle.dequantize_and_gather(want, w.k_cache.cpu(), seq.cpu(), None, table.cpu(), 64)
    assert torch.equal(out.cpu().view(torch.int16), want.view(torch.int16))


def test_host_checks_without_gpu():
    out = torch.zeros(2, 4, 512, dtype=torch.bfloat16)
    kc = torch.zeros(4, 64 * 584, dtype=torch.uint8)
    seq = torch.tensor([3, 4], dtype=torch.int32)
    table = torch.zeros(2, 1, dtype=torch.int32)
    with pytest.raises(AssertionError, match="no CPU path"):
        flaggems_vllm.dequantize_and_gather_k_cache(out, kc, seq, None, table, 64)
    with pytest.raises(AssertionError):
        flaggems_vllm.dequantize_and_gather_k_cache(out.float(), kc, seq, None, table, 64)
    with pytest.raises(AssertionError):
        flaggems_vllm.dequantize_and_gather_k_cache(out, kc, torch.zeros(3, dtype=torch.int32), None, table, 64)
    with pytest.raises(ValueError):
        flaggems_vllm.dequantize_and_gather_k_cache(out, kc.view(-1), seq, None, table, 64)
