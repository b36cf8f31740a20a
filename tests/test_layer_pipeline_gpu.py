"""The operators in the order a DeepSeek-V4 attention layer calls them, on one set of paged caches:
weighted norms -> activation quantiser -> (a stand-in for the q up-projection) -> prologue -> cache reader -> top-k
selection (on stand-in logits) -> index bookkeeping -> epilogue, and the sparse-indexer branch (q prologue, key insert,
key gather).  Each stage is checked against its oracle fed
with the previous stage's DEVICE result, so that a mismatch names the stage; then the whole chain is captured in a
CUDA graph and its replay compared with the eager run bit for bit."""
from __future__ import annotations

import pytest
import torch

import flaggems_vllm as fg
from flaggems_vllm.testing import compare, workloads
from oracle import c_oracle

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
HEADS, BS, EPS = 16, 64, 1e-6


def make_inputs(seed=0):
    g = torch.Generator().manual_seed(seed)
    seq_lens = [200, 64, 333]  # three requests, prefilled in one step
    n = sum(seq_lens)
    blocks_per_req = [-(-s // BS) for s in seq_lens]
    perm = torch.randperm(sum(blocks_per_req) + 2, generator=g).to(torch.int32)
    table = torch.full((3, max(blocks_per_req)), 0, dtype=torch.int32)
    at = 0
    for r, nb in enumerate(blocks_per_req):
        table[r, :nb] = perm[at : at + nb]
        at += nb
    positions = torch.cat([torch.arange(s) for s in seq_lens]).to(torch.int64)
    req_of = torch.cat([torch.full((s,), r) for r, s in enumerate(seq_lens)])
    slots = (table[req_of, (positions // BS)].to(torch.int64) * BS + positions % BS).contiguous()
    return {
        "n": n, "seq_lens": torch.tensor(seq_lens, dtype=torch.int32), "table": table, "positions": positions, "slots": slots,
        "req_of": req_of.to(torch.int32),
        "qr": torch.randn(n, 1536, generator=g).to(torch.bfloat16), "kv": torch.randn(n, 512, generator=g).to(torch.bfloat16),
        "wq": (1 + 0.1 * torch.randn(1536, generator=g)).to(torch.bfloat16), "wkv": (1 + 0.1 * torch.randn(512, generator=g)).to(torch.bfloat16),
        "up": (torch.randn(1536, HEADS * 512, generator=g) / 39.0).to(torch.bfloat16),
        "cs": workloads.cos_sin_table(4096),
        "iq": torch.randn(n, 8, 128, generator=g).to(torch.bfloat16), "iw": torch.randn(n, 8, generator=g).to(torch.bfloat16),
        "ik": torch.randn(n, 128, generator=g).to(torch.bfloat16),
        "cu": torch.tensor([0] + torch.cumsum(torch.tensor(seq_lens), 0).tolist(), dtype=torch.int32),
        "logits": torch.randn(n, 384, generator=g),  # stand-in for the indexer's MQA logits over each request's keys
        "row_ends": torch.cat([torch.arange(1, s + 1) for s in seq_lens]).to(torch.int32),  # causal: token i sees i + 1 keys
        "num_blocks": int(perm.numel()),
    }


def run_chain(d, buffers):
    """Every device-side stage; outputs that the operators allocate are returned, in-place ones live in `buffers`."""
    qr_n, kv_n = fg.fused_q_kv_rmsnorm(d["qr"], d["kv"], d["wq"], d["wkv"], EPS)
    q = (qr_n @ d["up"]).view(d["n"], HEADS, 512)  # stand-in for wq_b
    fg.fused_deepseek_v4_qnorm_rope_kv_rope_quant_insert(q, kv_n, buffers["k_cache"], d["slots"], d["positions"], d["cs"], EPS, BS)
    fg.dequantize_and_gather_k_cache(buffers["gathered"], buffers["k_cache"], d["seq_lens"], None, d["table"], BS)
    qr_fp8, qr_scale = fg.per_token_group_quant_fp8(qr_n, 128, scale_ue8m0=True)  # what the FP8 up-projection would consume
    fg.top_k_per_row_prefill(d["logits"], buffers["row_starts"], d["row_ends"], buffers["topk"], d["n"], d["logits"].stride(0), 1, 32)
    slots_topk, lens = fg.compute_global_topk_indices_and_lens(buffers["topk"], d["req_of"], d["table"], BS)
    fp8, scale = fg.fused_inv_rope_fp8_quant(q, d["positions"], d["cs"], 4, HEADS // 4, tma_aligned_scales=True)  # q stands in for o
    iq8, iw = fg.fused_indexer_q_rope_quant(d["positions"], d["iq"], d["cs"], d["iw"], 0.0884, 0.3536)
    fg.indexer_k_quant_and_cache(d["ik"], buffers["i_cache"], d["slots"], 128, "ue8m0")
    fg.cp_gather_indexer_k_quant_cache(buffers["i_cache"], buffers["ik8"], buffers["iks"], d["table"], d["cu"])
    return {"qr_n": qr_n, "kv_n": kv_n, "q": q, "qr_fp8": qr_fp8, "qr_scale": qr_scale, "slots_topk": slots_topk, "lens": lens, "fp8": fp8, "scale": scale, "iq8": iq8, "iw": iw}


def fresh_buffers(d):
    return {
        "k_cache": torch.zeros(d["num_blocks"], BS * 584, dtype=torch.uint8, device=DEV),
        "gathered": torch.zeros(3, 384, 512, dtype=torch.bfloat16, device=DEV),
        "i_cache": torch.zeros(d["num_blocks"], BS, 132, dtype=torch.uint8, device=DEV),
        "ik8": torch.zeros(d["n"], 128, dtype=torch.uint8, device=DEV), "iks": torch.zeros(d["n"], 4, dtype=torch.uint8, device=DEV),
        "topk": torch.zeros(d["n"], 32, dtype=torch.int32, device=DEV), "row_starts": torch.zeros(d["n"], dtype=torch.int32, device=DEV),
    }


def to_device(host):
    return {k: (v.to(DEV) if torch.is_tensor(v) else v) for k, v in host.items()}


def test_every_stage_matches_its_oracle():
    host = make_inputs()
    d = to_device(host)
    buffers = fresh_buffers(d)
    out = run_chain(d, buffers)
    torch.cuda.synchronize()
    cpu = lambda t: t.detach().cpu()
    # norms
    for got, x, w in ((out["qr_n"], host["qr"], host["wq"]), (out["kv_n"], host["kv"], host["wkv"])):
        assert int(compare.bf16_ulp_distance(cpu(got), c_oracle.weighted_rmsnorm(x, w, EPS)).max()) <= 1
    # prologue, from the device's own normalised kv and projected q
    q_in = (cpu(out["qr_n"]).to(DEV) @ d["up"]).view(d["n"], HEADS, 512).cpu()
    want_cache = torch.zeros(host["num_blocks"], BS * 584, dtype=torch.uint8)
    c_oracle.prologue(q_in, cpu(out["kv_n"]), want_cache, host["slots"], host["positions"], host["cs"], EPS, BS)
    assert torch.equal(cpu(buffers["k_cache"]), want_cache)
    compare.assert_q_close(cpu(out["q"]), q_in)
    # cache reader
    want_g = torch.zeros(3, 384, 512, dtype=torch.bfloat16)
    c_oracle.dequantize_and_gather(want_g, want_cache, host["seq_lens"], None, host["table"], BS)
    assert torch.equal(cpu(buffers["gathered"]).view(torch.int16), want_g.view(torch.int16))
    # activation quantiser on the device's normalised activations
    want_b, want_sc = c_oracle.per_token_group_quant_fp8(cpu(out["qr_n"]), 128, scale_ue8m0=True)
    assert torch.equal(cpu(out["qr_fp8"]).view(torch.uint8), want_b) and torch.equal(cpu(out["qr_scale"]).view(torch.int32), want_sc.view(torch.int32))
    # top-k selection: the values behind the selected positions, row by row, against the sorting oracle
    topk = cpu(buffers["topk"])
    ref = torch.zeros_like(topk)
    c_oracle.top_k_per_row_prefill(host["logits"], torch.zeros(host["n"], dtype=torch.int32), host["row_ends"], ref, host["n"], 384, 1, 32)
    for r in range(host["n"]):
        k = min(32, int(host["row_ends"][r]))
        assert bool((topk[r, k:] == -1).all()) and topk[r, :k].unique().numel() == k
        assert torch.equal(host["logits"][r, topk[r, :k].long()].sort().values, host["logits"][r, ref[r, :k].long()].sort().values)
    # index bookkeeping on the device's top-k: the slots are the slots the prologue wrote those positions to
    want_slots, want_lens = c_oracle.compute_global_topk_indices_and_lens(topk, host["req_of"], host["table"], BS)
    assert torch.equal(cpu(out["slots_topk"]), want_slots) and torch.equal(cpu(out["lens"]), want_lens)
    first_of_req = host["cu"][:-1].long()[host["req_of"].long()]
    picked = topk >= 0
    assert torch.equal(want_slots.long()[picked], host["slots"][(first_of_req[:, None] + topk.long())[picked]])
    assert torch.equal(want_lens.long(), host["row_ends"].long().clamp(max=32))
    # epilogue on the device's q
    want_fp8, want_scale = c_oracle.inv_rope_fp8_quant(cpu(out["q"]), host["positions"], host["cs"], 4, HEADS // 4, packed=True)
    assert torch.equal(cpu(out["fp8"]).view(torch.uint8), want_fp8)
    assert torch.equal(cpu(out["scale"]).contiguous().view(torch.int32), want_scale.view(torch.int32))
    # sparse-indexer branch
    want_q8, _, want_w = c_oracle.indexer_q_rope_quant(host["positions"], host["iq"], host["cs"], host["iw"], 0.0884, 0.3536)
    assert torch.equal(cpu(out["iq8"]).view(torch.uint8), want_q8) and torch.equal(cpu(out["iw"]), want_w)
    want_ic = torch.zeros(host["num_blocks"], BS, 132, dtype=torch.uint8)
    c_oracle.indexer_k_quant_and_cache(host["ik"], want_ic, host["slots"], 128, "ue8m0")
    assert torch.equal(cpu(buffers["i_cache"]), want_ic)
    want_k8, want_ks = torch.zeros(host["n"], 128, dtype=torch.uint8), torch.zeros(host["n"], 4, dtype=torch.uint8)
    c_oracle.cp_gather_indexer_k_quant_cache(want_ic, want_k8, want_ks, host["table"], host["cu"])
    assert torch.equal(cpu(buffers["ik8"]), want_k8) and torch.equal(cpu(buffers["iks"]), want_ks)


def test_chain_replays_from_a_cuda_graph():
    """No stage synchronises, reads back or allocates outside torch's caching allocator, so the chain is capturable;
    the replay must reproduce the eager results bit for bit (the top-k positions as sets: their order is not defined)."""
    d = to_device(make_inputs(seed=1))
    eager_buffers = fresh_buffers(d)
    eager = run_chain(d, eager_buffers)
    torch.cuda.synchronize()
    buffers = fresh_buffers(d)
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        run_chain(d, buffers)  # warm-up on the capture stream
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=s):
            captured = run_chain(d, buffers)
        for b in buffers.values():
            b.zero_()
        for t in captured.values():
            t.zero_()
        graph.replay()
    s.synchronize()
    raw = lambda t: t.view(torch.uint8) if t.dtype.itemsize == 1 else t  # float8 tensors compare as bytes
    # the top-k selection returns its positions in no particular order (as the reference's kernels do): rows as sets
    unordered = lambda k, t: t.sort(dim=1).values if k in ("slots_topk", "topk") else t
    for k in eager:
        assert torch.equal(unordered(k, raw(captured[k])), unordered(k, raw(eager[k]))), k
    for k in buffers:
        assert torch.equal(unordered(k, buffers[k]), unordered(k, eager_buffers[k])), k
