"""ctypes binding of libdsv4_prologue.so (the C ABI declared in include/dsv4_prologue.h).

There is no fallback: if the library has not been built, or a call is made on a
machine without a CUDA device, the caller gets an exception, never a silent
CPU or eager-PyTorch substitute.
"""
from __future__ import annotations

import ctypes
from pathlib import Path

LIB_NAME = "libdsv4_prologue.so"
LIB_PATH = Path(__file__).resolve().parent / LIB_NAME

EXPORTS = (
    "dsv4_qnorm_rope_kv_insert",
    "dsv4_qnorm_rope_kv_insert_checked",
    "dsv4_qnorm_rope_kv_insert_padded",
    "dsv4_gather_dequant_k_cache",
    "dsv4_dequantize_and_gather_k_cache",
    "dsv4_fused_q_kv_rmsnorm",
    "dsv4_fused_q_kv_rmsnorm_dtypes",
    "dsv4_fused_inv_rope_fp8_quant",
    "dsv4_fused_inv_rope_fp8_quant_geometry",
    "dsv4_indexer_k_quant_and_cache",
    "dsv4_cp_gather_indexer_k_quant_cache",
    "dsv4_compute_global_topk_indices_and_lens",
    "dsv4_combine_topk_swa_indices",
    "dsv4_per_token_group_quant_fp8",
    "dsv4_act_quant",
    "dsv4_top_k_per_row_decode",
    "dsv4_top_k_per_row_prefill",
    "dsv4_fused_indexer_q_rope_quant",
    "dsv4_device_error",
    "dsv4_set_variant",
    "dsv4_get_variant",
    "dsv4_set_bulk_wait_cycles",
    "dsv4_bulk_wait_selftest",
    "dsv4_set_pdl",
    "dsv4_set_table_staging",
    "dsv4_launch_count",
    "dsv4_error_string",
    "dsv4_version",
)

VARIANT_AUTO, VARIANT_ROWS, VARIANT_BULK = 0, 1, 2

_lib = None


class NativeLibraryMissing(RuntimeError):
    pass


class Dsv4Error(RuntimeError):
    def __init__(self, code: int, text: str):
        super().__init__(f"libdsv4_prologue: {text} (code {code})")
        self.code = code


def lib() -> ctypes.CDLL:
    """Load (once) and return the library; raises NativeLibraryMissing if it was never built."""
    global _lib
    if _lib is not None:
        return _lib
    if not LIB_PATH.exists():
        raise NativeLibraryMissing(
            f"{LIB_PATH} is missing: build it with `python -m flaggems_vllm.build` "
            "(nvcc, sm_100a). This package has no CPU or PyTorch fallback."
        )
    L = ctypes.CDLL(str(LIB_PATH))
    vp, i64, i32, f32 = ctypes.c_void_p, ctypes.c_int64, ctypes.c_int, ctypes.c_float
    L.dsv4_qnorm_rope_kv_insert.argtypes = [vp, vp, vp, vp, vp, vp, f32, i64, i64, i64, i64, i64, vp]
    L.dsv4_qnorm_rope_kv_insert.restype = i32
    L.dsv4_qnorm_rope_kv_insert_checked.argtypes = [vp, vp, vp, vp, vp, vp, f32, i64, i64, i64, i64, i64,
                                                    i64, i64, vp, vp]
    L.dsv4_qnorm_rope_kv_insert_checked.restype = i32
    L.dsv4_qnorm_rope_kv_insert_padded.argtypes = [vp, vp, vp, vp, vp, vp, vp, f32, i64, i64, i64, i64, i64, i64, vp]
    L.dsv4_qnorm_rope_kv_insert_padded.restype = i32
    L.dsv4_gather_dequant_k_cache.argtypes = [vp, vp, i64, vp, i64, i64, i64, vp]
    L.dsv4_gather_dequant_k_cache.restype = i32
    L.dsv4_dequantize_and_gather_k_cache.argtypes = [vp, i64, i64, i64, vp, vp, vp, vp, i64, i64, i64, i64, i64,
                                                     i32, i32, i32, i32, vp]
    L.dsv4_dequantize_and_gather_k_cache.restype = i32
    L.dsv4_fused_q_kv_rmsnorm.argtypes = [vp, vp, vp, i64, i64, i64, vp, vp, vp, i64, i64, i64, i64, f32, vp]
    L.dsv4_fused_q_kv_rmsnorm.restype = i32
    L.dsv4_fused_q_kv_rmsnorm_dtypes.argtypes = [vp, vp, vp, i64, i64, i64, i32, i32, vp, vp, vp, i64, i64, i64, i32, i32, i64, f32, vp]
    L.dsv4_fused_q_kv_rmsnorm_dtypes.restype = i32
    L.dsv4_fused_inv_rope_fp8_quant.argtypes = [vp, i64, i64, vp, vp, i64, vp, vp, i64, i64, i64, i64, i64, f32, i32, vp]
    L.dsv4_fused_inv_rope_fp8_quant.restype = i32
    L.dsv4_fused_inv_rope_fp8_quant_geometry.argtypes = [vp, i64, i64, vp, vp, i64, vp, vp, i64, i64, i64, i64, i64, i64, i64, i64, f32, i32, vp]
    L.dsv4_fused_inv_rope_fp8_quant_geometry.restype = i32
    L.dsv4_indexer_k_quant_and_cache.argtypes = [vp, i64, i32, vp, i64, vp, i64, i64, i64, i64, i32, vp]
    L.dsv4_indexer_k_quant_and_cache.restype = i32
    L.dsv4_cp_gather_indexer_k_quant_cache.argtypes = [vp, i64, vp, i64, vp, i64, vp, i64, vp, i64, i64, i64, i64, i64, vp]
    L.dsv4_cp_gather_indexer_k_quant_cache.restype = i32
    L.dsv4_compute_global_topk_indices_and_lens.argtypes = [vp, i64, vp, vp, i64, vp, vp, i64, vp, i64, i64, i64, vp]
    L.dsv4_compute_global_topk_indices_and_lens.restype = i32
    L.dsv4_combine_topk_swa_indices.argtypes = [vp, i64, i64, vp, vp, vp, vp, i64, i64, vp, i64, i64, i64, i64, i64, i64, i64, vp]
    L.dsv4_combine_topk_swa_indices.restype = i32
    L.dsv4_per_token_group_quant_fp8.argtypes = [vp, i64, vp, vp, i64, i64, i64, i64, i64, f32, i32, vp]
    L.dsv4_per_token_group_quant_fp8.restype = i32
    L.dsv4_act_quant.argtypes = [vp, i64, vp, vp, i64, i64, i64, i32, vp]
    L.dsv4_act_quant.restype = i32
    L.dsv4_top_k_per_row_decode.argtypes = [vp, i64, i64, i64, vp, vp, i64, i64, i64, vp]
    L.dsv4_top_k_per_row_decode.restype = i32
    L.dsv4_top_k_per_row_prefill.argtypes = [vp, i64, i64, vp, vp, vp, i64, i64, i64, vp]
    L.dsv4_top_k_per_row_prefill.restype = i32
    L.dsv4_fused_indexer_q_rope_quant.argtypes = [vp, vp, i64, i64, vp, i64, i32, i64, vp, i64, i64, vp, i64, i64, vp, i64, i32,
                                                  vp, i64, f32, f32, i64, i64, i64, i32, vp]
    L.dsv4_fused_indexer_q_rope_quant.restype = i32
    L.dsv4_device_error.argtypes = [vp]
    L.dsv4_device_error.restype = i32
    L.dsv4_set_pdl.argtypes = [i32]
    L.dsv4_set_pdl.restype = i32
    L.dsv4_set_bulk_wait_cycles.argtypes = [i64]
    L.dsv4_set_bulk_wait_cycles.restype = i64
    L.dsv4_bulk_wait_selftest.argtypes = [vp, vp, vp, vp, vp, vp, f32, i64, i64, i64, i64, i64, i64, vp]
    L.dsv4_bulk_wait_selftest.restype = i32
    L.dsv4_set_table_staging.argtypes = [i32]
    L.dsv4_set_table_staging.restype = i32
    L.dsv4_set_variant.argtypes = [i32]
    L.dsv4_set_variant.restype = i32
    L.dsv4_get_variant.restype = i32
    L.dsv4_launch_count.restype = i64
    L.dsv4_error_string.argtypes = [i32]
    L.dsv4_error_string.restype = ctypes.c_char_p
    L.dsv4_version.restype = ctypes.c_char_p
    _lib = L
    return L


def check(code: int) -> None:
    if code != 0:
        raise Dsv4Error(code, lib().dsv4_error_string(code).decode())


def device_error() -> int:
    """Read and clear the current device's kernel error word (synchronises); 0 = healthy."""
    v = ctypes.c_int32(0)
    check(lib().dsv4_device_error(ctypes.byref(v)))
    return int(v.value)


def launch_count() -> int:
    return int(lib().dsv4_launch_count())


def set_variant(variant: int) -> int:
    prev = lib().dsv4_set_variant(int(variant))
    if prev < 0:
        raise Dsv4Error(prev, lib().dsv4_error_string(prev).decode())
    return prev


def set_pdl(mode) -> int:
    """Programmatic dependent launch of the prologue (see dsv4_set_pdl): 0 / False off, 1 / True with early index
    reads, 2 with ordinary stream semantics; returns the previous mode."""
    return int(lib().dsv4_set_pdl(int(mode)))


def set_table_staging(mode: int) -> int:
    """-1: by launch size, 0: per-warp table fetch, 1: shared-memory staging (see dsv4_set_table_staging);
    returns the previous mode."""
    return int(lib().dsv4_set_table_staging(int(mode)))


def version() -> str:
    return lib().dsv4_version().decode()
