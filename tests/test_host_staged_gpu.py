"""The host-buffer front end (pinned host tensors in, rewritten q out, copies overlapped with the kernel) gives
the same q and the same cache as one device-resident call."""
from __future__ import annotations

import pytest
import torch

import flaggems_vllm
from flaggems_vllm.testing import workloads

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


@pytest.mark.parametrize("num_tokens,chunk,depth,n_insert", [(1000, 256, 3, 1000), (777, 100, 2, 700), (64, 1024, 3, 64), (513, 64, 4, 0)])
def test_matches_device_resident_call(num_tokens, chunk, depth, n_insert):
    w = workloads.make("cpu_ref", device=DEV, seed=21, num_tokens=num_tokens, num_heads=8, num_blocks=32)
    slots = w.slot_mapping[:n_insert].contiguous()
    slots[::13] = -1
    q_ref, cache_ref = w.q.clone(), w.k_cache.clone()
    flaggems_vllm.fused_deepseek_v4_qnorm_rope_kv_rope_quant_insert(q_ref, w.kv, cache_ref, slots, w.position_ids,
                                                                  w.cos_sin_cache, w.eps, 64)
    hq, hkv = w.q.cpu().pin_memory(), w.kv.cpu().pin_memory()
    hslots, hpos = slots.cpu().pin_memory(), w.position_ids.cpu().pin_memory()
    pipe = flaggems_vllm.HostStagedPrologue(8, chunk_tokens=chunk, device=DEV, depth=depth)
    out = torch.empty_like(hq).pin_memory()
    for _ in range(2):  # the second pass reuses every staging buffer
        cache = w.k_cache.clone()
        res = pipe(hq, hkv, cache, hslots, hpos, w.cos_sin_cache, w.eps, 64, q_out_host=out)
        assert res is out
        assert torch.equal(out.view(torch.int16), q_ref.cpu().view(torch.int16))
        assert torch.equal(cache, cache_ref)
        assert pipe.launches == (num_tokens + chunk - 1) // chunk
    # in place on the host buffer
    cache = w.k_cache.clone()
    pipe(hq, hkv, cache, hslots, hpos, w.cos_sin_cache, w.eps, 64)
    assert torch.equal(hq.view(torch.int16), q_ref.cpu().view(torch.int16)) and torch.equal(cache, cache_ref)
