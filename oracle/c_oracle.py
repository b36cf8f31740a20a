"""ctypes front end of the C oracle (`dsv4_oracle.c`).  TEST INFRASTRUCTURE ONLY.

All tensors are CPU tensors.  The library is built by `oracle/Makefile`
(`build()` below runs it); nothing here touches a GPU.
"""
from __future__ import annotations

import ctypes
import os
import subprocess
from pathlib import Path

import torch

_DIR = Path(__file__).resolve().parent
_LIB_PATH = _DIR / "libdsv4_oracle.so"
_lib = None


def build(force: bool = False) -> Path:
    """Compile the oracle with the Makefile beside it (gcc, OpenMP, no FP contraction)."""
    src = _DIR / "dsv4_oracle.c"
    if force or not _LIB_PATH.exists() or _LIB_PATH.stat().st_mtime < src.stat().st_mtime:
        subprocess.run(["make", "-C", str(_DIR), "-B"], check=True, capture_output=True)
    return _LIB_PATH


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        build()
        L = ctypes.CDLL(str(_LIB_PATH))
        i64, vp, f32, i32 = ctypes.c_int64, ctypes.c_void_p, ctypes.c_float, ctypes.c_int
        L.dsv4_oracle_prologue.argtypes = [vp, vp, vp, vp, vp, vp, f32, i64, i64, i64, i64, i64, i32]
        L.dsv4_oracle_prologue.restype = i32
        L.dsv4_oracle_gather_dequant.argtypes = [vp, vp, i64, vp, i64, i64, i32]
        L.dsv4_oracle_gather_dequant.restype = i32
        for name in ("dsv4_oracle_bf16_from_f32", "dsv4_oracle_e4m3_from_f32", "dsv4_oracle_f32_from_e4m3"):
            getattr(L, name).argtypes = [vp, vp, i64]
            getattr(L, name).restype = None
        L.dsv4_oracle_ue8m0_codes.argtypes = [vp, vp, vp, i64]
        L.dsv4_oracle_ue8m0_codes.restype = None
        L.dsv4_oracle_dequantize_and_gather.argtypes = [vp, i64, i64, vp, vp, vp, vp, i64, i64, i64, i64, i64, i32, i32, i32]
        L.dsv4_oracle_dequantize_and_gather.restype = i32
        L.dsv4_oracle_weighted_rmsnorm.argtypes = [vp, vp, vp, i64, i64, i64, i64, f32]
        L.dsv4_oracle_weighted_rmsnorm.restype = i32
        L.dsv4_oracle_inv_rope_fp8_quant.argtypes = [vp, i64, i64, vp, vp, i64, vp, vp, i64, i64, i64, f32, i32]
        L.dsv4_oracle_inv_rope_fp8_quant.restype = i32
        L.dsv4_oracle_inv_rope_fp8_quant_geometry.argtypes = [vp, i64, i64, vp, vp, i64, vp, vp, i64, i64, i64, i64, i64, i64, f32, i32]
        L.dsv4_oracle_inv_rope_fp8_quant_geometry.restype = i32
        L.dsv4_oracle_indexer_k_quant.argtypes = [vp, i64, i32, vp, i64, vp, i64, i64, i64, i64, i32]
        L.dsv4_oracle_indexer_k_quant.restype = i32
        L.dsv4_oracle_cp_gather_indexer.argtypes = [vp, i64, vp, i64, vp, i64, vp, i64, vp, i64, i64, i64, i64, i64]
        L.dsv4_oracle_cp_gather_indexer.restype = i32
        L.dsv4_oracle_global_topk.argtypes = [vp, i64, vp, vp, i64, vp, vp, i64, vp, i64, i64, i64]
        L.dsv4_oracle_global_topk.restype = i32
        L.dsv4_oracle_combine_topk_swa.argtypes = [vp, i64, i64, vp, vp, vp, vp, i64, i64, vp, i64, i64, i64, i64, i64, i64, i64]
        L.dsv4_oracle_combine_topk_swa.restype = i32
        L.dsv4_oracle_top_k_per_row.argtypes = [vp, i64, i64, vp, vp, vp, i64, i64, i64]
        L.dsv4_oracle_top_k_per_row.restype = i32
        L.dsv4_oracle_group_quant_fp8.argtypes = [vp, i64, vp, vp, i64, i64, i64, i64, i64, f32, i32, i32]
        L.dsv4_oracle_group_quant_fp8.restype = i32
        L.dsv4_oracle_indexer_q_rope_quant.argtypes = [vp, vp, vp, i64, vp, f32, f32, i64, i64, i64, i32, vp, vp, vp]
        L.dsv4_oracle_indexer_q_rope_quant.restype = i32
        L.dsv4_oracle_check_division_shortcut.argtypes = [f32, i32, i32, vp, vp]
        L.dsv4_oracle_check_division_shortcut.restype = i64
        L.dsv4_oracle_version.restype = ctypes.c_char_p
        _lib = L
    return _lib


def _cpu(t: torch.Tensor, dtype: torch.dtype) -> torch.Tensor:
    assert t.device.type == "cpu" and t.dtype == dtype and t.is_contiguous(), (t.device, t.dtype)
    return t


def prologue(q, kv, k_cache, slot_mapping, position_ids, cos_sin_cache, eps, cache_block_size, threads=0) -> None:
    """Same arguments and in-place effects as the operator, on CPU tensors."""
    _cpu(q, torch.bfloat16), _cpu(kv, torch.bfloat16), _cpu(k_cache, torch.uint8)
    _cpu(slot_mapping, torch.int64), _cpu(position_ids, torch.int64), _cpu(cos_sin_cache, torch.float32)
    n, h, d = q.shape
    assert d == 512 and kv.shape == (n, 512) and k_cache.dim() == 2
    rc = lib().dsv4_oracle_prologue(
        q.data_ptr(), kv.data_ptr(), k_cache.data_ptr(), slot_mapping.data_ptr(), position_ids.data_ptr(),
        cos_sin_cache.data_ptr(), float(eps), n, h, slot_mapping.shape[0], int(cache_block_size),
        k_cache.stride(0), int(threads or os.cpu_count() or 1),
    )
    if rc != 0:
        raise ValueError(f"dsv4_oracle_prologue rejected its arguments (rc={rc})")


def gather_dequant(k_cache, slots, cache_block_size, threads=0) -> torch.Tensor:
    """bf16 [len(slots), 512]: the de-quantised cached tokens at `slots`."""
    _cpu(k_cache, torch.uint8), _cpu(slots, torch.int64)
    out = torch.empty(slots.shape[0], 512, dtype=torch.bfloat16)
    rc = lib().dsv4_oracle_gather_dequant(
        k_cache.data_ptr(), slots.data_ptr(), slots.shape[0], out.data_ptr(), int(cache_block_size),
        k_cache.stride(0), int(threads or os.cpu_count() or 1),
    )
    if rc != 0:
        raise ValueError(f"dsv4_oracle_gather_dequant rejected its arguments (rc={rc})")
    return out


def dequantize_and_gather(out, k_cache, seq_lens, gather_lens, block_table, block_size, offset=0, rope_dim=64,
                          nope_dim=None, scale_slots=None) -> None:
    """Same arguments as the reference operator, on CPU tensors (int32 index tensors); fills `out`."""
    _cpu(k_cache, torch.uint8), _cpu(seq_lens, torch.int32), _cpu(block_table, torch.int32)
    assert out.dtype == torch.bfloat16 and out.dim() == 3 and out.stride(2) == 1 and k_cache.dim() == 2
    nope_dim = out.shape[-1] - rope_dim if nope_dim is None else nope_dim
    scale_slots = (nope_dim + 63) // 64 + (1 if nope_dim % 64 == 0 else 0) if scale_slots is None else scale_slots
    gl = None if gather_lens is None else _cpu(gather_lens, torch.int32).data_ptr()
    rc = lib().dsv4_oracle_dequantize_and_gather(
        out.data_ptr(), out.stride(0), out.stride(1), k_cache.data_ptr(), seq_lens.data_ptr(), gl, block_table.data_ptr(),
        seq_lens.shape[0], block_table.shape[1], int(block_size), k_cache.stride(0), int(offset), int(nope_dim),
        int(rope_dim), int(scale_slots))
    if rc != 0:
        raise ValueError("dsv4_oracle_dequantize_and_gather rejected its arguments")


def weighted_rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """bf16 [rows, size] -> (x * rsqrt(mean(x^2) + eps)) * weight, fp32 arithmetic."""
    assert x.dtype == torch.bfloat16 and x.dim() == 2 and x.stride(1) == 1 and x.device.type == "cpu"
    _cpu(weight, torch.bfloat16)
    out = torch.empty(x.shape, dtype=torch.bfloat16)
    rc = lib().dsv4_oracle_weighted_rmsnorm(x.data_ptr(), weight.data_ptr(), out.data_ptr(), x.shape[0], x.shape[1],
                                            x.stride(0), out.stride(0), float(eps))
    if rc != 0:
        raise ValueError("dsv4_oracle_weighted_rmsnorm rejected its arguments")
    return out


def inv_rope_fp8_quant(o, positions, cos_sin_cache, n_groups, heads_per_group, eps=1e-10, packed=False, nope_dim=448, rope_dim=64,
                       quant_group_size=128):
    """(fp8 bytes uint8 [N, G, hpg*head_dim], scales [N, G, hpg*K] fp32 or [N, G, hpg] int32; K = groups per head) on
    CPU tensors."""
    head_dim = nope_dim + rope_dim
    assert o.dtype == torch.bfloat16 and o.dim() == 3 and o.shape[2] == head_dim and o.stride(2) == 1 and o.device.type == "cpu"
    _cpu(positions, torch.int64), _cpu(cos_sin_cache, torch.float32)
    n = o.shape[0]
    assert o.shape[1] == n_groups * heads_per_group and head_dim % quant_group_size == 0
    chunks = head_dim // quant_group_size
    fp8 = torch.empty(n, n_groups, heads_per_group * head_dim, dtype=torch.uint8)
    scales = torch.empty(n, n_groups, heads_per_group * (1 if packed else chunks), dtype=torch.int32 if packed else torch.float32)
    rc = lib().dsv4_oracle_inv_rope_fp8_quant_geometry(o.data_ptr(), o.stride(0), o.stride(1), positions.data_ptr(),
                                                       cos_sin_cache.data_ptr(), cos_sin_cache.stride(0), fp8.data_ptr(),
                                                       scales.data_ptr(), n, n_groups, heads_per_group, int(nope_dim), int(rope_dim),
                                                       int(quant_group_size), float(eps), 1 if packed else 0)
    if rc != 0:
        raise ValueError("dsv4_oracle_inv_rope_fp8_quant rejected its arguments")
    return fp8, scales


def indexer_k_quant_and_cache(k, kv_cache, slot_mapping, quant_block_size, scale_fmt) -> None:
    """Same arguments as the reference operator, on CPU tensors; kv_cache [blocks, block_size, row] uint8 in place."""
    assert k.device.type == "cpu" and k.dim() == 2 and k.stride(1) == 1 and k.dtype in (torch.bfloat16, torch.float16)
    _cpu(kv_cache, torch.uint8), _cpu(slot_mapping, torch.int64)
    rc = lib().dsv4_oracle_indexer_k_quant(k.data_ptr(), k.stride(0), 1 if k.dtype == torch.float16 else 0, kv_cache.data_ptr(),
                                           kv_cache.stride(0), slot_mapping.data_ptr(), slot_mapping.shape[0], kv_cache.shape[1],
                                           k.shape[1], int(quant_block_size), 1 if scale_fmt == "ue8m0" else 0)
    if rc != 0:
        raise ValueError("dsv4_oracle_indexer_k_quant rejected its arguments")


def cp_gather_indexer_k_quant_cache(k_cache, k_fp8, k_fp8_scale, block_table, cu_seqlen) -> None:
    """Same arguments as the reference operator, on CPU tensors; k_fp8 [T, head_dim] (1-byte elements) and k_fp8_scale
    [T, 4*groups bytes] are written in place for the tokens inside a request."""
    _cpu(k_cache, torch.uint8), _cpu(block_table, torch.int32), _cpu(cu_seqlen, torch.int32)
    assert k_cache.dim() == 3 and k_cache.is_contiguous() and k_fp8.device.type == "cpu" and k_fp8_scale.device.type == "cpu"
    assert k_fp8.element_size() == 1 and k_fp8.stride(1) == 1 and k_fp8_scale.stride(1) == 1 and block_table.stride(1) == 1
    head_dim = k_fp8.shape[1]
    scale_bytes = k_fp8_scale.shape[1] * k_fp8_scale.element_size()
    assert scale_bytes % 4 == 0 and k_cache.shape[2] == head_dim + scale_bytes
    rc = lib().dsv4_oracle_cp_gather_indexer(k_cache.data_ptr(), k_cache.stride(0), k_fp8.data_ptr(), k_fp8.stride(0),
                                             k_fp8_scale.data_ptr(), k_fp8_scale.stride(0) * k_fp8_scale.element_size(),
                                             block_table.data_ptr(), block_table.stride(0), cu_seqlen.data_ptr(),
                                             block_table.shape[0], k_fp8.shape[0], k_cache.shape[1], head_dim, scale_bytes // 4)
    if rc != 0:
        raise ValueError("dsv4_oracle_cp_gather_indexer rejected its arguments")


def compute_global_topk_indices_and_lens(topk_indices, token_to_req_indices, block_table, block_size, is_valid_token=None):
    """Same arguments and return values as the reference operator, on CPU int32 tensors."""
    for t in (topk_indices, token_to_req_indices, block_table) + (() if is_valid_token is None else (is_valid_token,)):
        _cpu(t, torch.int32)
    assert topk_indices.dim() == 2 and topk_indices.stride(1) == 1 and block_table.stride(1) == 1
    out = torch.empty_like(topk_indices, dtype=torch.int32)
    lens = torch.empty(topk_indices.shape[0], dtype=torch.int32)
    rc = lib().dsv4_oracle_global_topk(topk_indices.data_ptr(), topk_indices.stride(0), token_to_req_indices.contiguous().data_ptr(),
                                       block_table.data_ptr(), block_table.stride(0),
                                       None if is_valid_token is None else is_valid_token.contiguous().data_ptr(), out.data_ptr(),
                                       out.stride(0), lens.data_ptr(), topk_indices.shape[0], topk_indices.shape[1], int(block_size))
    if rc != 0:
        raise ValueError("dsv4_oracle_global_topk rejected its arguments")
    return out, lens


def combine_topk_swa_indices(topk_indices, query_start_loc, seq_lens, gather_lens, window_size, compress_ratio, topk, M, N, fill=None):
    """Same arguments and return values as the reference operator, on CPU int32 tensors.  Rows that no request covers
    keep `fill` (the reference leaves them uninitialised)."""
    for t in (topk_indices, query_start_loc, seq_lens, gather_lens):
        _cpu(t, torch.int32)
    assert topk_indices.dim() == 2 and topk_indices.stride(1) == 1
    width = (topk + window_size + 127) // 128 * 128
    tokens = topk_indices.shape[0]
    combined = torch.full((tokens, width), 0 if fill is None else fill, dtype=torch.int32)
    lens = torch.full((tokens,), 0 if fill is None else fill, dtype=torch.int32)
    rc = lib().dsv4_oracle_combine_topk_swa(topk_indices.data_ptr(), topk_indices.stride(0), topk_indices.shape[1],
                                            query_start_loc.contiguous().data_ptr(), seq_lens.contiguous().data_ptr(),
                                            gather_lens.contiguous().data_ptr(), combined.data_ptr(), combined.stride(0), width,
                                            lens.data_ptr(), seq_lens.shape[0], tokens, int(window_size), int(compress_ratio), int(topk),
                                            int(M), int(N))
    if rc != 0:
        raise ValueError("dsv4_oracle_combine_topk_swa rejected its arguments")
    return combined, lens


def top_k_per_row_prefill(logits, row_starts, row_ends, indices, num_rows, stride0, stride1, top_k) -> None:
    """Same arguments as the reference operator, on CPU tensors; fills `indices` [num_rows, top_k] int32."""
    _cpu(row_starts, torch.int32), _cpu(row_ends, torch.int32), _cpu(indices, torch.int32)
    assert logits.device.type == "cpu" and logits.dtype == torch.float32  # any strides
    assert indices.is_contiguous() and indices.shape[1] == top_k and logits.dim() == 2 and num_rows == logits.shape[0]
    rc = lib().dsv4_oracle_top_k_per_row(logits.data_ptr(), logits.stride(0), logits.stride(1), row_starts.contiguous().data_ptr(),
                                         row_ends.contiguous().data_ptr(), indices.data_ptr(), num_rows, logits.shape[1], int(top_k))
    if rc != 0:
        raise ValueError("dsv4_oracle_top_k_per_row rejected its arguments")


def top_k_per_row_decode(logits, next_n, seq_lens, indices, num_rows, stride0, stride1, top_k) -> None:
    """Same arguments as the reference operator, on CPU tensors: row i covers [0, seq_lens[i // next_n] - next_n + i % next_n + 1)."""
    rows = torch.arange(num_rows)
    ends = (seq_lens.to(torch.int64)[rows // next_n] - next_n + rows % next_n + 1).to(torch.int32)
    top_k_per_row_prefill(logits, torch.zeros(num_rows, dtype=torch.int32), ends, indices, num_rows, stride0, stride1, top_k)


def per_token_group_quant_fp8(x, group_size, eps=1e-10, column_major_scales=False, scale_ue8m0=False, act_quant_rules=False):
    """(bytes uint8 shaped like x, scales fp32 [M, K / group_size]) on a CPU bf16 tensor [M, K] with unit inner stride;
    `column_major_scales` returns the scales with transposed storage, as the reference does."""
    assert x.device.type == "cpu" and x.dtype == torch.bfloat16 and x.dim() == 2 and x.stride(1) == 1
    rows, cols = x.shape
    out = torch.empty(rows, cols, dtype=torch.uint8)
    groups = cols // group_size
    scales = torch.empty(groups, rows).permute(1, 0) if column_major_scales else torch.empty(rows, groups)
    rc = lib().dsv4_oracle_group_quant_fp8(x.data_ptr(), x.stride(0), out.data_ptr(), scales.data_ptr(), scales.stride(0), scales.stride(1),
                                           rows, cols, int(group_size), float(eps), 1 if scale_ue8m0 else 0, 1 if act_quant_rules else 0)
    if rc != 0:
        raise ValueError("dsv4_oracle_group_quant_fp8 rejected its arguments")
    return out, scales


def act_quant(x, block_size=128, scale_fmt=None):
    """(bytes uint8, scales fp32) of the reference's `act_quant_triton` on a CPU bf16 tensor [M, N]."""
    return per_token_group_quant_fp8(x, block_size, eps=1e-4, scale_ue8m0=scale_fmt is not None, act_quant_rules=True)


def indexer_q_rope_quant(positions, index_q, cos_sin_cache, weights, softmax_scale, head_scale, use_fp4=False):
    """(q bytes uint8, scales uint8 or None, weights_out fp32) on CPU tensors; cos_sin_cache and weights of any float dtype."""
    _cpu(positions, torch.int64)
    q = _cpu(index_q.contiguous(), torch.bfloat16)
    cs = cos_sin_cache.float().contiguous()
    w = weights.float().contiguous()
    t, h, d = q.shape
    out = torch.empty(t, h, d // 2 if use_fp4 else d, dtype=torch.uint8)
    scales = torch.empty(t, h, d // 32, dtype=torch.uint8) if use_fp4 else None
    w_out = torch.empty(t, h, dtype=torch.float32)
    rc = lib().dsv4_oracle_indexer_q_rope_quant(positions.data_ptr(), q.data_ptr(), cs.data_ptr(), cs.shape[1], w.data_ptr(),
                                                float(softmax_scale), float(head_scale), t, h, d, 1 if use_fp4 else 0,
                                                out.data_ptr(), scales.data_ptr() if use_fp4 else None, w_out.data_ptr())
    if rc != 0:
        raise ValueError("dsv4_oracle_indexer_q_rope_quant rejected its arguments")
    return out, scales, w_out


def check_division_shortcut(eps: float = 1e-10, form: int = 3, y_ulps: int = 0):
    """(pairs examined, e4m3 byte mismatches, fp32 value mismatches) of the CUDA quantisers' division shortcut:
    form 2 = two-term reciprocal (scales up to 2^100), form 3 = product with one correction (any scale); `y_ulps`
    moves the reciprocal off RN(1/scale) by that many ulps (the device's reciprocal is within one)."""
    b, v = ctypes.c_int64(0), ctypes.c_int64(0)
    n = lib().dsv4_oracle_check_division_shortcut(float(eps), int(form), int(y_ulps), ctypes.byref(b), ctypes.byref(v))
    return int(n), int(b.value), int(v.value)


def e4m3_from_f32(x: torch.Tensor) -> torch.Tensor:
    x = _cpu(x.contiguous(), torch.float32)
    out = torch.empty(x.shape, dtype=torch.uint8)
    lib().dsv4_oracle_e4m3_from_f32(x.data_ptr(), out.data_ptr(), x.numel())
    return out


def f32_from_e4m3(b: torch.Tensor) -> torch.Tensor:
    b = _cpu(b.contiguous(), torch.uint8)
    out = torch.empty(b.shape, dtype=torch.float32)
    lib().dsv4_oracle_f32_from_e4m3(b.data_ptr(), out.data_ptr(), b.numel())
    return out


def bf16_from_f32(x: torch.Tensor) -> torch.Tensor:
    x = _cpu(x.contiguous(), torch.float32)
    out = torch.empty(x.shape, dtype=torch.bfloat16)
    lib().dsv4_oracle_bf16_from_f32(x.data_ptr(), out.data_ptr(), x.numel())
    return out


def ue8m0_codes(amax: torch.Tensor):
    """(codes by the log2/ceil statement, codes by the bit-pattern derivation)."""
    amax = _cpu(amax.contiguous(), torch.float32)
    a = torch.empty(amax.shape, dtype=torch.uint8)
    b = torch.empty(amax.shape, dtype=torch.uint8)
    lib().dsv4_oracle_ue8m0_codes(amax.data_ptr(), a.data_ptr(), b.data_ptr(), amax.numel())
    return a, b
