"""The slot-addressed cache reader against its CPU oracle, and the write -> read round trip."""
from __future__ import annotations

import pytest
import torch

import flaggems_vllm
from flaggems_vllm.testing import workloads
from oracle import c_oracle

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


@pytest.mark.parametrize("block_size,stride_pad,offset", [(64, 0, 0), (16, 0, 0), (16, 64, 0), (16, 8, 0), (16, 0, 5)])
def test_reader_matches_oracle_on_arbitrary_bytes(block_size, stride_pad, offset):
    """Any byte pattern is a valid cache row except the e4m3 NaN codes; compare bit patterns."""
    g = torch.Generator().manual_seed(block_size + stride_pad + offset)
    nb, pitch = 9, block_size * 584 + stride_pad
    kc = torch.randint(0, 256, (nb, pitch), generator=g, dtype=torch.uint8)
    kc[(kc & 0x7F) == 0x7F] = 0x3C  # no NaN codes: NaN payloads are not comparable bit for bit
    scales = kc[:, block_size * 576 : block_size * 584]
    scales.copy_(torch.randint(100, 140, scales.shape, generator=g, dtype=torch.uint8))
    slots = torch.randperm(nb * block_size, generator=g)[:100].to(torch.int64)
    slots[::9] = -1
    backing = torch.zeros(nb * pitch + 32, dtype=torch.uint8, device=DEV)
    view = backing[offset : offset + nb * pitch].view(nb, pitch)
    view.copy_(kc)
    out = flaggems_vllm.gather_dequant_k_cache_slots(view, slots.to(DEV), block_size)
    want = c_oracle.gather_dequant(kc, slots, block_size)
    assert torch.equal(out.cpu().view(torch.int16), want.view(torch.int16))


def test_write_then_read_round_trip_at_prefill_size():
    """prologue -> reader on 8192 tokens: RoPE part returns exactly what the oracle caches, the
    de-quantised part is within the e4m3 step of the original kv."""
    w = workloads.make("prefill", device=DEV, seed=2, num_heads=1)
    flaggems_vllm.fused_deepseek_v4_qnorm_rope_kv_rope_quant_insert(*w.args())
    rows = flaggems_vllm.gather_dequant_k_cache_slots(w.k_cache, w.slot_mapping, 64)
    torch.cuda.synchronize()
    small = torch.zeros(w.num_tokens // 64 + 1, 64 * 584, dtype=torch.uint8)
    compact = torch.arange(w.num_tokens)
    c_oracle.prologue(torch.empty(w.num_tokens, 0, 512, dtype=torch.bfloat16), w.kv.cpu(), small, compact,
                      w.position_ids.cpu(), w.cos_sin_cache.cpu(), w.eps, 64)
    want = c_oracle.gather_dequant(small, compact, 64)
    assert torch.equal(rows.cpu().view(torch.int16), want.view(torch.int16))
    kvf, got = w.kv[:, :448].float(), rows[:, :448].float()
    amax = kvf.view(-1, 7, 64).abs().amax(dim=-1, keepdim=True).clamp(min=1e-4)
    step = torch.exp2(torch.ceil(torch.log2(amax / 448.0)))  # scale; e4m3 subnormal step is scale * 2^-9
    err = (got - kvf).view(-1, 7, 64).abs()
    assert bool((err <= kvf.view(-1, 7, 64).abs() * 2.0 ** -4 + step * 2.0 ** -10).all())
