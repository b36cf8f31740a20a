// extern "C" surface of libdsv4_prologue.so: argument validation, variant choice, launch.
// Declarations and the reference interface each entry point replaces: include/dsv4_prologue.h.
#include <atomic>
#include <cstdlib>

#include "../../include/dsv4_prologue.h"
#include "dsv4_common.cuh"

namespace dsv4 {
namespace {
std::atomic<int64_t> g_launches{0};
std::atomic<int> g_variant{-1};  // -1: not initialised from the environment yet
std::atomic<int> g_pdl{-1};      // programmatic dependent launch of the rows variant; -1: not initialised yet

int current_variant() {
    int v = g_variant.load(std::memory_order_relaxed);
    if (v < 0) {
        v = DSV4_VARIANT_AUTO;
        if (const char* e = std::getenv("DSV4_VARIANT")) {
            const int parsed = std::atoi(e);
            if (parsed >= DSV4_VARIANT_AUTO && parsed <= DSV4_VARIANT_BULK) v = parsed;
        }
        g_variant.store(v, std::memory_order_relaxed);
    }
    return v;
}

int current_pdl() {
    int v = g_pdl.load(std::memory_order_relaxed);
    if (v < 0) {
        const char* e = std::getenv("DSV4_PDL");
        v = e ? std::atoi(e) : 2;
        if (v < 0 || v > 2) v = 2;
        g_pdl.store(v, std::memory_order_relaxed);
    }
    return v;
}

// Where the rows variant takes the cos|sin rows from: -1 = by launch size (per-warp fetch up to kPerWarpTableRows rows
// of q, shared-memory staging above), 0 = always per warp, 1 = always staged.
std::atomic<int> g_table_staging{-2};  // -2: not initialised from the environment yet
constexpr int64_t kPerWarpTableRows = 65536;

int current_table_staging() {
    int v = g_table_staging.load(std::memory_order_relaxed);
    if (v < -1) {
        const char* e = std::getenv("DSV4_TABLE_STAGING");
        v = e ? std::atoi(e) : -1;
        if (v < -1 || v > 1) v = -1;
        g_table_staging.store(v, std::memory_order_relaxed);
    }
    return v;
}

// Bulk variant: SM cycles a wait on a shared-memory barrier may take before the kernel gives up.  A tile load is a few
// microseconds; 2e8 cycles are about a tenth of a second at B200 clocks.
std::atomic<long long> g_bulk_wait_cycles{200000000LL};

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// `any_alignment`: where given, q and kv only need their element's 2-byte alignment and the table its 4 bytes, and
// *any_alignment says whether the launch has to take the kernel for such pointers; where NULL, 16 bytes are required.
int validate(const void* q, const void* kv, const void* k_cache, const int64_t* slot_mapping,
             const int64_t* position_ids, const float* cos_sin_cache, int64_t num_tokens, int64_t num_heads,
             int64_t num_tokens_insert, int64_t cache_block_size, int64_t kv_block_stride_bytes, bool* any_alignment = nullptr) {
    if (any_alignment) *any_alignment = false;
    if (num_tokens < 0 || num_heads < 0 || num_tokens_insert < 0 || num_tokens_insert > num_tokens)
        return DSV4_ERR_BAD_SIZE;
    if (num_tokens == 0) return DSV4_OK;
    if (!position_ids || !cos_sin_cache) return DSV4_ERR_NULL_POINTER;
    if (num_heads > 0 && !q) return DSV4_ERR_NULL_POINTER;
    if (num_tokens_insert > 0) {
        if (!kv || !k_cache || !slot_mapping) return DSV4_ERR_NULL_POINTER;
        if (cache_block_size <= 0 || kv_block_stride_bytes < cache_block_size * (kTokenDataBytes + kScaleBytes))
            return DSV4_ERR_BAD_SIZE;
    }
    if (!aligned16(q) || !aligned16(kv) || !aligned16(cos_sin_cache)) {
        const auto low_bits = [](const void* p, uintptr_t mask) { return (reinterpret_cast<uintptr_t>(p) & mask) != 0; };
        if (!any_alignment || low_bits(q, 1u) || low_bits(kv, 1u) || low_bits(cos_sin_cache, 3u)) return DSV4_ERR_MISALIGNED;
        *any_alignment = true;
    }
    // kernels index q rows and tokens with 32 bits (2^31 rows of 1 KiB are 2 TiB, beyond any GPU)
    if (num_tokens >= (1LL << 31) || num_heads >= (1LL << 31)) return DSV4_ERR_TOO_LARGE;
    if (num_heads > 0 && num_tokens > ((1LL << 31) - 1) / num_heads) return DSV4_ERR_TOO_LARGE;
    return DSV4_OK;
}

PrologueParams make_params(void* q, const void* kv, void* k_cache, const int64_t* slot_mapping,
                           const int64_t* position_ids, const float* cos_sin_cache, float eps, int64_t num_tokens,
                           int64_t num_heads, int64_t num_tokens_insert, int64_t cache_block_size,
                           int64_t kv_block_stride_bytes) {
    PrologueParams p{};
    p.q = static_cast<uint8_t*>(q);
    p.kv = static_cast<const uint8_t*>(kv);
    p.k_cache = static_cast<uint8_t*>(k_cache);
    p.slot_mapping = slot_mapping;
    p.position_ids = position_ids;
    p.cos_sin = cos_sin_cache;
    p.eps = eps;
    p.num_tokens = num_tokens;
    p.num_heads = num_heads;
    p.num_tokens_insert = num_tokens_insert;
    p.block_size = cache_block_size > 0 ? cache_block_size : 1;
    p.block_stride = kv_block_stride_bytes;
    p.cache_aligned16 = aligned16(k_cache) && (kv_block_stride_bytes % 16 == 0);
    make_fast_divisor(static_cast<uint32_t>(num_heads > 0 ? num_heads : 1), &p.heads_mul, &p.heads_shift);
    p.pdl = current_pdl();
    p.wait_cycles = g_bulk_wait_cycles.load(std::memory_order_relaxed);
    p.short_tile = 0xffffffffu;
    const int staging = current_table_staging();
    p.table_staging = staging < 0 ? (num_tokens * num_heads > kPerWarpTableRows ? 1 : 0) : staging;
    return p;
}
}  // namespace

void count_launch() { g_launches.fetch_add(1, std::memory_order_relaxed); }
}  // namespace dsv4

using namespace dsv4;

extern "C" {

int dsv4_qnorm_rope_kv_insert(void* q, const void* kv, void* k_cache, const int64_t* slot_mapping,
                              const int64_t* position_ids, const float* cos_sin_cache, float eps,
                              int64_t num_tokens, int64_t num_heads, int64_t num_tokens_insert,
                              int64_t cache_block_size, int64_t kv_block_stride_bytes, void* cuda_stream) {
    bool any_alignment = false;
    const int rc = validate(q, kv, k_cache, slot_mapping, position_ids, cos_sin_cache, num_tokens, num_heads,
                            num_tokens_insert, cache_block_size, kv_block_stride_bytes, &any_alignment);
    if (rc != DSV4_OK || num_tokens == 0) return rc;
    const PrologueParams p = make_params(q, kv, k_cache, slot_mapping, position_ids, cos_sin_cache, eps, num_tokens,
                                         num_heads, num_tokens_insert, cache_block_size, kv_block_stride_bytes);
    cudaStream_t stream = static_cast<cudaStream_t>(cuda_stream);
    if (any_alignment) return static_cast<int>(launch_prologue_rows_any_alignment(p, stream));
    int variant = current_variant();
    if (variant == DSV4_VARIANT_AUTO) variant = DSV4_VARIANT_ROWS;
    const cudaError_t err = variant == DSV4_VARIANT_BULK ? launch_prologue_bulk(p, stream)
                                                         : launch_prologue_rows(p, false, stream);
    return static_cast<int>(err);
}

int dsv4_qnorm_rope_kv_insert_padded(const void* q, void* q_out, const void* kv, void* k_cache, const int64_t* slot_mapping,
                                     const int64_t* position_ids, const float* cos_sin_cache, float eps, int64_t num_tokens,
                                     int64_t num_heads, int64_t padded_heads, int64_t num_tokens_insert,
                                     int64_t cache_block_size, int64_t kv_block_stride_bytes, void* cuda_stream) {
    const int rc = validate(q, kv, k_cache, slot_mapping, position_ids, cos_sin_cache, num_tokens, num_heads,
                            num_tokens_insert, cache_block_size, kv_block_stride_bytes);
    if (rc != DSV4_OK || num_tokens == 0) return rc;
    if (padded_heads < num_heads || padded_heads >= (1LL << 31) || num_tokens > ((1LL << 31) - 1) / (padded_heads > 0 ? padded_heads : 1))
        return DSV4_ERR_BAD_SIZE;
    if (padded_heads > 0 && !q_out) return DSV4_ERR_NULL_POINTER;
    if (!aligned16(q_out)) return DSV4_ERR_MISALIGNED;
    PrologueParams p = make_params(const_cast<void*>(q), kv, k_cache, slot_mapping, position_ids, cos_sin_cache, eps, num_tokens,
                                   num_heads, num_tokens_insert, cache_block_size, kv_block_stride_bytes);
    p.q_out = static_cast<uint8_t*>(q_out);
    p.out_heads = padded_heads;
    return static_cast<int>(launch_prologue_rows_padded(p, static_cast<cudaStream_t>(cuda_stream)));
}

int dsv4_qnorm_rope_kv_insert_checked(void* q, const void* kv, void* k_cache, const int64_t* slot_mapping,
                                      const int64_t* position_ids, const float* cos_sin_cache, float eps,
                                      int64_t num_tokens, int64_t num_heads, int64_t num_tokens_insert,
                                      int64_t cache_block_size, int64_t kv_block_stride_bytes,
                                      int64_t num_blocks, int64_t max_pos, int32_t* status, void* cuda_stream) {
    const int rc = validate(q, kv, k_cache, slot_mapping, position_ids, cos_sin_cache, num_tokens, num_heads,
                            num_tokens_insert, cache_block_size, kv_block_stride_bytes);
    if (rc != DSV4_OK || num_tokens == 0) return rc;
    if (!status) return DSV4_ERR_NULL_POINTER;
    if (num_blocks < 0 || max_pos < 0) return DSV4_ERR_BAD_SIZE;
    PrologueParams p = make_params(q, kv, k_cache, slot_mapping, position_ids, cos_sin_cache, eps, num_tokens,
                                   num_heads, num_tokens_insert, cache_block_size, kv_block_stride_bytes);
    p.num_slots = num_blocks * p.block_size;
    p.max_pos = max_pos;
    p.status = status;
    return static_cast<int>(launch_prologue_rows(p, true, static_cast<cudaStream_t>(cuda_stream)));
}

int dsv4_gather_dequant_k_cache(const void* k_cache, const int64_t* slots, int64_t num_slots, void* out,
                                int64_t out_row_stride, int64_t cache_block_size,
                                int64_t kv_block_stride_bytes, void* cuda_stream) {
    if (num_slots < 0 || out_row_stride < kHeadDim) return DSV4_ERR_BAD_SIZE;
    if (num_slots == 0) return DSV4_OK;
    if (!k_cache || !slots || !out) return DSV4_ERR_NULL_POINTER;
    if (cache_block_size <= 0 || kv_block_stride_bytes < cache_block_size * (kTokenDataBytes + kScaleBytes))
        return DSV4_ERR_BAD_SIZE;
    if (!aligned16(out) || (out_row_stride % 8) != 0) return DSV4_ERR_MISALIGNED;
    return static_cast<int>(launch_gather_dequant(static_cast<const uint8_t*>(k_cache), slots, num_slots,
                                                  static_cast<uint8_t*>(out), out_row_stride, cache_block_size,
                                                  kv_block_stride_bytes, static_cast<cudaStream_t>(cuda_stream)));
}

int dsv4_dequantize_and_gather_k_cache(void* out, int64_t out_stride0, int64_t out_stride1, int64_t out_tokens,
                                       const void* k_cache, const void* seq_lens, const void* gather_lens,
                                       const void* block_table, int64_t num_reqs, int64_t max_blocks_per_seq,
                                       int64_t cache_block_size, int64_t kv_block_stride_bytes, int64_t offset,
                                       int32_t nope_dim, int32_t rope_dim, int32_t scale_slots, int32_t index_is_int64,
                                       void* cuda_stream) {
    if (num_reqs < 0 || out_tokens < 0 || offset < 0 || nope_dim < 0 || rope_dim < 0 || scale_slots < 0)
        return DSV4_ERR_BAD_SIZE;
    if (num_reqs == 0 || out_tokens == 0) return DSV4_OK;
    if (!out || !k_cache || !seq_lens || !block_table) return DSV4_ERR_NULL_POINTER;
    if (cache_block_size <= 0 || max_blocks_per_seq <= 0 || scale_slots * 64 < nope_dim) return DSV4_ERR_BAD_SIZE;
    if (kv_block_stride_bytes < cache_block_size * (nope_dim + 2 * rope_dim + scale_slots)) return DSV4_ERR_BAD_SIZE;
    if (num_reqs > 65535) return DSV4_ERR_TOO_LARGE;
    if ((reinterpret_cast<uintptr_t>(out) & 1u) != 0) return DSV4_ERR_MISALIGNED;
    return static_cast<int>(launch_gather_dequant_requests(
        static_cast<uint8_t*>(out), out_stride0, out_stride1, static_cast<const uint8_t*>(k_cache), seq_lens, gather_lens,
        block_table, num_reqs, max_blocks_per_seq, cache_block_size, kv_block_stride_bytes, offset, nope_dim, rope_dim,
        scale_slots, index_is_int64 ? 1 : 0, out_tokens, static_cast<cudaStream_t>(cuda_stream)));
}

int dsv4_fused_q_kv_rmsnorm(const void* qr, void* qr_out, const void* q_weight, int64_t q_in_stride,
                            int64_t q_out_stride, int64_t q_size, const void* kv, void* kv_out, const void* kv_weight,
                            int64_t kv_in_stride, int64_t kv_out_stride, int64_t kv_size, int64_t num_tokens, float eps,
                            void* cuda_stream) {
    if (num_tokens < 0 || q_size <= 0 || kv_size <= 0 || q_size >= (1LL << 31) || kv_size >= (1LL << 31))
        return DSV4_ERR_BAD_SIZE;
    if (num_tokens == 0) return DSV4_OK;
    if (!qr || !qr_out || !q_weight || !kv || !kv_out || !kv_weight) return DSV4_ERR_NULL_POINTER;
    const auto odd = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 1u) != 0; };
    if (odd(qr) || odd(qr_out) || odd(q_weight) || odd(kv) || odd(kv_out) || odd(kv_weight)) return DSV4_ERR_MISALIGNED;
    return static_cast<int>(launch_q_kv_rmsnorm(qr, qr_out, q_weight, q_in_stride, q_out_stride, q_size, kv, kv_out,
                                                kv_weight, kv_in_stride, kv_out_stride, kv_size, num_tokens, eps,
                                                static_cast<cudaStream_t>(cuda_stream)));
}

int dsv4_fused_q_kv_rmsnorm_dtypes(const void* qr, void* qr_out, const void* q_weight, int64_t q_in_stride, int64_t q_out_stride,
                                   int64_t q_size, int32_t q_dtype, int32_t q_weight_dtype, const void* kv, void* kv_out,
                                   const void* kv_weight, int64_t kv_in_stride, int64_t kv_out_stride, int64_t kv_size,
                                   int32_t kv_dtype, int32_t kv_weight_dtype, int64_t num_tokens, float eps, void* cuda_stream) {
    if (num_tokens < 0 || q_size <= 0 || kv_size <= 0 || q_size >= (1LL << 31) || kv_size >= (1LL << 31))
        return DSV4_ERR_BAD_SIZE;
    for (const int32_t d : {q_dtype, q_weight_dtype, kv_dtype, kv_weight_dtype})
        if (d < 0 || d > 2) return DSV4_ERR_BAD_SIZE;
    if (num_tokens == 0) return DSV4_OK;
    if (!qr || !qr_out || !q_weight || !kv || !kv_out || !kv_weight) return DSV4_ERR_NULL_POINTER;
    const auto misaligned = [](const void* p, int32_t dtype) { return (reinterpret_cast<uintptr_t>(p) & (dtype == 2 ? 3u : 1u)) != 0; };
    if (misaligned(qr, q_dtype) || misaligned(qr_out, q_dtype) || misaligned(q_weight, q_weight_dtype) || misaligned(kv, kv_dtype) ||
        misaligned(kv_out, kv_dtype) || misaligned(kv_weight, kv_weight_dtype))
        return DSV4_ERR_MISALIGNED;
    if (q_dtype == 0 && q_weight_dtype == 0 && kv_dtype == 0 && kv_weight_dtype == 0)
        return dsv4_fused_q_kv_rmsnorm(qr, qr_out, q_weight, q_in_stride, q_out_stride, q_size, kv, kv_out, kv_weight, kv_in_stride,
                                       kv_out_stride, kv_size, num_tokens, eps, cuda_stream);
    return static_cast<int>(launch_q_kv_rmsnorm_any(qr, qr_out, q_weight, q_in_stride, q_out_stride, q_size, q_dtype, q_weight_dtype, kv,
                                                    kv_out, kv_weight, kv_in_stride, kv_out_stride, kv_size, kv_dtype, kv_weight_dtype,
                                                    num_tokens, eps, static_cast<cudaStream_t>(cuda_stream)));
}

int dsv4_fused_inv_rope_fp8_quant(const void* o, int64_t o_stride_token, int64_t o_stride_head, const int64_t* positions,
                                  const float* cos_sin_cache, int64_t cos_sin_stride, void* fp8_out, void* scale_out,
                                  int64_t scale_stride_group, int64_t num_tokens, int64_t padded_tokens, int64_t n_groups,
                                  int64_t heads_per_group, float eps, int32_t packed_ue8m0_scales, void* cuda_stream) {
    if (num_tokens < 0 || padded_tokens < num_tokens || padded_tokens % 4 != 0 || n_groups <= 0 || heads_per_group <= 0 ||
        n_groups * heads_per_group >= (1LL << 31))
        return DSV4_ERR_BAD_SIZE;
    if (num_tokens == 0) return DSV4_OK;
    if (!o || !positions || !cos_sin_cache || !fp8_out || !scale_out) return DSV4_ERR_NULL_POINTER;
    if (!aligned16(o) || !aligned16(cos_sin_cache) || o_stride_token % 8 != 0 || o_stride_head % 8 != 0 ||
        cos_sin_stride % 4 != 0 || (reinterpret_cast<uintptr_t>(fp8_out) & 7u) != 0 ||
        (reinterpret_cast<uintptr_t>(scale_out) & 3u) != 0)
        return DSV4_ERR_MISALIGNED;
    return static_cast<int>(launch_inv_rope_fp8_quant(o, o_stride_token, o_stride_head, positions, cos_sin_cache, cos_sin_stride,
                                                      fp8_out, scale_out, scale_stride_group, num_tokens, padded_tokens,
                                                      static_cast<int>(n_groups * heads_per_group),
                                                      static_cast<int>(heads_per_group), eps, packed_ue8m0_scales ? 1 : 0,
                                                      static_cast<cudaStream_t>(cuda_stream)));
}

int dsv4_fused_inv_rope_fp8_quant_geometry(const void* o, int64_t o_stride_token, int64_t o_stride_head, const int64_t* positions,
                                           const float* cos_sin_cache, int64_t cos_sin_stride, void* fp8_out, void* scale_out,
                                           int64_t scale_stride_group, int64_t num_tokens, int64_t padded_tokens, int64_t n_groups,
                                           int64_t heads_per_group, int64_t nope_dim, int64_t rope_dim, int64_t quant_group_size,
                                           float eps, int32_t packed_ue8m0_scales, void* cuda_stream) {
    if (num_tokens < 0 || padded_tokens < num_tokens || padded_tokens % 4 != 0 || n_groups <= 0 || heads_per_group <= 0 ||
        n_groups * heads_per_group >= (1LL << 31))
        return DSV4_ERR_BAD_SIZE;
    // the reference wrapper's geometry rules (src/flaggems_vllm/ops/fused_inv_rope_fp8_quant.py:193-200), plus an even group
    const int64_t head_dim = nope_dim + rope_dim;
    if (nope_dim < 0 || rope_dim < 0 || quant_group_size <= 0 || head_dim <= 0 || head_dim >= (1 << 20) || head_dim % quant_group_size != 0 ||
        nope_dim % quant_group_size != quant_group_size - rope_dim || rope_dim % 2 != 0 || quant_group_size % 2 != 0)
        return DSV4_ERR_BAD_SIZE;
    if (packed_ue8m0_scales && head_dim / quant_group_size != 4) return DSV4_ERR_BAD_SIZE;
    const bool fast_layout = aligned16(o) && aligned16(cos_sin_cache) && o_stride_token % 8 == 0 && o_stride_head % 8 == 0 &&
                             cos_sin_stride % 4 == 0 && (reinterpret_cast<uintptr_t>(fp8_out) & 7u) == 0;
    if (nope_dim == 448 && rope_dim == 64 && quant_group_size == 128 && (fast_layout || num_tokens == 0))
        return dsv4_fused_inv_rope_fp8_quant(o, o_stride_token, o_stride_head, positions, cos_sin_cache, cos_sin_stride, fp8_out,
                                             scale_out, scale_stride_group, num_tokens, padded_tokens, n_groups, heads_per_group, eps,
                                             packed_ue8m0_scales, cuda_stream);
    if (num_tokens == 0) return DSV4_OK;
    if (!o || !positions || !cos_sin_cache || !fp8_out || !scale_out) return DSV4_ERR_NULL_POINTER;
    const auto low_bits = [](const void* p, uintptr_t mask) { return (reinterpret_cast<uintptr_t>(p) & mask) != 0; };
    if (low_bits(o, 1u) || low_bits(cos_sin_cache, 3u) || low_bits(fp8_out, 1u) || low_bits(scale_out, 3u)) return DSV4_ERR_MISALIGNED;
    return static_cast<int>(launch_inv_rope_fp8_quant_any(
        o, o_stride_token, o_stride_head, positions, cos_sin_cache, cos_sin_stride, fp8_out, scale_out, scale_stride_group, num_tokens,
        padded_tokens, static_cast<int>(n_groups * heads_per_group), static_cast<int>(heads_per_group), static_cast<int>(nope_dim),
        static_cast<int>(rope_dim), static_cast<int>(quant_group_size), eps, packed_ue8m0_scales ? 1 : 0,
        static_cast<cudaStream_t>(cuda_stream)));
}

int dsv4_indexer_k_quant_and_cache(const void* k, int64_t k_row_stride, int32_t k_is_fp16, void* kv_cache,
                                   int64_t cache_block_stride_bytes, const int64_t* slot_mapping, int64_t num_tokens,
                                   int64_t cache_block_size, int64_t head_dim, int64_t quant_block_size,
                                   int32_t scale_is_ue8m0, void* cuda_stream) {
    if (num_tokens < 0 || head_dim <= 0 || quant_block_size <= 0 || head_dim % quant_block_size != 0 ||
        head_dim >= (1LL << 24) || cache_block_size <= 0)
        return DSV4_ERR_BAD_SIZE;
    if (num_tokens == 0) return DSV4_OK;
    if (!k || !kv_cache || !slot_mapping) return DSV4_ERR_NULL_POINTER;
    if (cache_block_stride_bytes < cache_block_size * (head_dim + 4 * (head_dim / quant_block_size))) return DSV4_ERR_BAD_SIZE;
    // the fp32 scale region of every block must be 4-byte aligned
    if ((reinterpret_cast<uintptr_t>(k) & 1u) != 0 || (reinterpret_cast<uintptr_t>(kv_cache) & 3u) != 0 ||
        cache_block_stride_bytes % 4 != 0 || (cache_block_size * head_dim) % 4 != 0)
        return DSV4_ERR_MISALIGNED;
    return static_cast<int>(launch_indexer_k_quant(k, k_row_stride, k_is_fp16 ? 1 : 0, kv_cache, cache_block_stride_bytes,
                                                   slot_mapping, num_tokens, cache_block_size, static_cast<int>(head_dim),
                                                   static_cast<int>(quant_block_size), scale_is_ue8m0 ? 1 : 0,
                                                   static_cast<cudaStream_t>(cuda_stream)));
}

int dsv4_cp_gather_indexer_k_quant_cache(const void* k_cache, int64_t cache_block_stride_bytes, void* k_out,
                                         int64_t k_out_stride_bytes, void* scale_out, int64_t scale_out_stride_bytes,
                                         const int32_t* block_table, int64_t block_table_stride, const int32_t* cu_seqlen,
                                         int64_t batch, int64_t num_tokens, int64_t cache_block_size, int64_t head_dim,
                                         int64_t num_quant_blocks, void* cuda_stream) {
    if (num_tokens < 0 || num_tokens >= (1LL << 31) || batch < 0 || batch >= (1LL << 31) - 1 || head_dim <= 0 ||
        head_dim >= (1LL << 24) || num_quant_blocks <= 0 || num_quant_blocks > head_dim || cache_block_size <= 0 ||
        cache_block_size >= (1LL << 31))
        return DSV4_ERR_BAD_SIZE;
    if (num_tokens == 0 || batch == 0) return DSV4_OK;
    if (!k_cache || !k_out || !scale_out || !block_table || !cu_seqlen) return DSV4_ERR_NULL_POINTER;
    if (cache_block_stride_bytes < cache_block_size * (head_dim + 4 * num_quant_blocks) || k_out_stride_bytes < head_dim ||
        scale_out_stride_bytes < 4 * num_quant_blocks)
        return DSV4_ERR_BAD_SIZE;
    return static_cast<int>(launch_cp_gather_indexer(k_cache, cache_block_stride_bytes, k_out, k_out_stride_bytes, scale_out,
                                                     scale_out_stride_bytes, block_table, block_table_stride, cu_seqlen, batch,
                                                     num_tokens, cache_block_size, static_cast<int>(head_dim),
                                                     static_cast<int>(num_quant_blocks), static_cast<cudaStream_t>(cuda_stream)));
}

int dsv4_compute_global_topk_indices_and_lens(const int32_t* topk_indices, int64_t topk_stride, const int32_t* token_to_req,
                                              const int32_t* block_table, int64_t block_table_stride, const int32_t* is_valid_token,
                                              int32_t* global_indices, int64_t global_stride, int32_t* lens, int64_t num_tokens,
                                              int64_t topk, int64_t block_size, void* cuda_stream) {
    if (num_tokens < 0 || topk < 0 || topk >= (1LL << 31) || block_size <= 0 || block_size >= (1LL << 31) || topk_stride < topk ||
        global_stride < topk)
        return DSV4_ERR_BAD_SIZE;
    if (num_tokens == 0) return DSV4_OK;
    if (!topk_indices || !token_to_req || !block_table || !global_indices || !lens) return DSV4_ERR_NULL_POINTER;
    return static_cast<int>(launch_global_topk(topk_indices, topk_stride, token_to_req, block_table, block_table_stride, is_valid_token,
                                               global_indices, global_stride, lens, num_tokens, static_cast<int>(topk),
                                               static_cast<int>(block_size), static_cast<cudaStream_t>(cuda_stream)));
}

int dsv4_combine_topk_swa_indices(const int32_t* topk_indices, int64_t topk_stride, int64_t topk_width,
                                  const int32_t* query_start_loc, const int32_t* seq_lens, const int32_t* gather_lens,
                                  int32_t* combined, int64_t combined_stride, int64_t combined_width, int32_t* lens,
                                  int64_t num_reqs, int64_t num_tokens, int64_t window_size, int64_t compress_ratio, int64_t topk,
                                  int64_t M, int64_t N, void* cuda_stream) {
    const int64_t lim = 1LL << 31;
    if (num_tokens < 0 || num_tokens >= lim || num_reqs < 0 || num_reqs >= lim - 1 || topk < 0 || topk > topk_width ||
        topk_width >= lim || window_size < 0 || compress_ratio <= 0 || compress_ratio >= lim || combined_width >= lim ||
        topk + window_size > combined_width || topk_stride < topk_width || combined_stride < combined_width || M <= -lim ||
        M >= lim || N <= -lim || N >= lim)
        return DSV4_ERR_BAD_SIZE;
    if (num_tokens == 0 || num_reqs == 0) return DSV4_OK;
    if (!topk_indices || !query_start_loc || !seq_lens || !gather_lens || !combined || !lens) return DSV4_ERR_NULL_POINTER;
    return static_cast<int>(launch_combine_topk_swa(topk_indices, topk_stride, static_cast<int>(topk_width), query_start_loc, seq_lens,
                                                    gather_lens, combined, combined_stride, static_cast<int>(combined_width), lens,
                                                    num_reqs, num_tokens, static_cast<int>(window_size),
                                                    static_cast<int>(compress_ratio), static_cast<int>(topk), static_cast<int>(M),
                                                    static_cast<int>(N), static_cast<cudaStream_t>(cuda_stream)));
}

namespace {
int check_topk_sizes(const float* logits, const int32_t* indices, int64_t num_rows, int64_t vocab, int64_t top_k) {
    const int64_t lim = 1LL << 31;
    if (num_rows < 0 || num_rows >= lim || vocab < 0 || vocab >= lim || top_k < 0 || top_k >= lim) return DSV4_ERR_BAD_SIZE;
    if (num_rows > 0 && top_k > 0 && (!logits || !indices)) return DSV4_ERR_NULL_POINTER;
    if ((reinterpret_cast<uintptr_t>(logits) & 3u) != 0 || (reinterpret_cast<uintptr_t>(indices) & 3u) != 0) return DSV4_ERR_MISALIGNED;
    return DSV4_OK;
}
}  // namespace

int dsv4_top_k_per_row_decode(const float* logits, int64_t stride0, int64_t stride1, int64_t next_n, const int32_t* seq_lens,
                              int32_t* indices, int64_t num_rows, int64_t vocab, int64_t top_k, void* cuda_stream) {
    const int rc = check_topk_sizes(logits, indices, num_rows, vocab, top_k);
    if (rc != DSV4_OK) return rc;
    if (next_n <= 0 || next_n >= (1LL << 31)) return DSV4_ERR_BAD_SIZE;
    if (num_rows == 0 || top_k == 0) return DSV4_OK;
    if (!seq_lens) return DSV4_ERR_NULL_POINTER;
    return static_cast<int>((vocab <= 8192 ? launch_topk_per_row_short : launch_topk_per_row)(logits, stride0, stride1, indices, num_rows, static_cast<int>(vocab),
                                                static_cast<int>(top_k), seq_lens, static_cast<int>(next_n), nullptr, nullptr,
                                                static_cast<cudaStream_t>(cuda_stream)));
}

int dsv4_top_k_per_row_prefill(const float* logits, int64_t stride0, int64_t stride1, const int32_t* row_starts,
                               const int32_t* row_ends, int32_t* indices, int64_t num_rows, int64_t vocab, int64_t top_k,
                               void* cuda_stream) {
    const int rc = check_topk_sizes(logits, indices, num_rows, vocab, top_k);
    if (rc != DSV4_OK) return rc;
    if (num_rows == 0 || top_k == 0) return DSV4_OK;
    if (!row_ends) return DSV4_ERR_NULL_POINTER;
    return static_cast<int>((vocab <= 8192 ? launch_topk_per_row_short : launch_topk_per_row)(logits, stride0, stride1, indices, num_rows, static_cast<int>(vocab),
                                                static_cast<int>(top_k), nullptr, 1, row_starts, row_ends,
                                                static_cast<cudaStream_t>(cuda_stream)));
}

namespace {
int group_quant(const void* x, int64_t x_row_stride, void* out, float* scales, int64_t scale_stride_row, int64_t scale_stride_group,
                int64_t num_rows, int64_t num_cols, int64_t group_size, float eps, int32_t scale_is_ue8m0, int act_quant_rules,
                void* cuda_stream) {
    if (num_rows < 0 || num_cols < 0 || group_size <= 0 || group_size >= (1LL << 24) || num_cols % group_size != 0 ||
        x_row_stride < num_cols)
        return DSV4_ERR_BAD_SIZE;
    if (num_rows == 0 || num_cols == 0) return DSV4_OK;
    if (!x || !out || !scales) return DSV4_ERR_NULL_POINTER;
    if ((reinterpret_cast<uintptr_t>(x) & 1u) != 0 || (reinterpret_cast<uintptr_t>(scales) & 3u) != 0) return DSV4_ERR_MISALIGNED;
    return static_cast<int>(launch_group_quant_fp8(x, x_row_stride, out, scales, scale_stride_row, scale_stride_group, num_rows, num_cols,
                                                   static_cast<int>(group_size), eps, scale_is_ue8m0 ? 1 : 0, act_quant_rules,
                                                   static_cast<cudaStream_t>(cuda_stream)));
}
}  // namespace

int dsv4_per_token_group_quant_fp8(const void* x, int64_t x_row_stride, void* out, float* scales, int64_t scale_stride_row,
                                   int64_t scale_stride_group, int64_t num_rows, int64_t num_cols, int64_t group_size, float eps,
                                   int32_t scale_is_ue8m0, void* cuda_stream) {
    return group_quant(x, x_row_stride, out, scales, scale_stride_row, scale_stride_group, num_rows, num_cols, group_size, eps,
                       scale_is_ue8m0, 0, cuda_stream);
}

int dsv4_act_quant(const void* x, int64_t x_row_stride, void* out, float* scales, int64_t num_rows, int64_t num_cols, int64_t block_size,
                   int32_t round_scale, void* cuda_stream) {
    return group_quant(x, x_row_stride, out, scales, block_size > 0 ? num_cols / block_size : 0, 1, num_rows, num_cols, block_size, 1e-4f,
                       round_scale, 1, cuda_stream);
}

int dsv4_fused_indexer_q_rope_quant(const int64_t* positions, const void* index_q, int64_t q_stride0, int64_t q_stride1,
                                    const void* cos_sin_cache, int64_t cos_sin_stride, int32_t cos_sin_is_bf16, int64_t rot_dim,
                                    void* q_out, int64_t out_stride0, int64_t out_stride1, void* q_scales_out,
                                    int64_t scale_stride0, int64_t scale_stride1, const void* weights, int64_t weights_stride,
                                    int32_t weights_dtype, float* weights_out, int64_t weights_out_stride, float softmax_scale,
                                    float head_scale, int64_t num_tokens, int64_t num_heads, int64_t head_dim, int32_t use_fp4,
                                    void* cuda_stream) {
    if (num_tokens < 0 || num_heads <= 0 || num_heads >= (1LL << 31)) return DSV4_ERR_BAD_SIZE;
    if (head_dim != 64 && head_dim != 128 && head_dim != 256) return DSV4_ERR_BAD_SIZE;
    const int64_t lane_elems = head_dim / 32;
    if (rot_dim < 0 || rot_dim > head_dim || rot_dim % 2 != 0 || (head_dim - rot_dim) % lane_elems != 0) return DSV4_ERR_BAD_SIZE;
    if (weights_dtype < 0 || weights_dtype > 2) return DSV4_ERR_BAD_SIZE;
    if (num_tokens == 0) return DSV4_OK;
    if (!positions || !index_q || (!cos_sin_cache && rot_dim > 0) || !q_out || !weights || !weights_out ||
        (use_fp4 && !q_scales_out))
        return DSV4_ERR_NULL_POINTER;
    const auto addr = [](const void* p) { return reinterpret_cast<uintptr_t>(p); };
    const int64_t in_bytes = lane_elems * 2, out_bytes = use_fp4 ? lane_elems / 2 : lane_elems;
    if (addr(index_q) % in_bytes || (q_stride0 * 2) % in_bytes || (q_stride1 * 2) % in_bytes || addr(q_out) % out_bytes ||
        out_stride0 % out_bytes || out_stride1 % out_bytes || addr(cos_sin_cache) % (cos_sin_is_bf16 ? 2 : 4) ||
        addr(weights_out) % 4)
        return DSV4_ERR_MISALIGNED;
    return static_cast<int>(launch_indexer_q_rope_quant(
        positions, index_q, q_stride0, q_stride1, cos_sin_cache, cos_sin_stride, cos_sin_is_bf16 ? 1 : 0, static_cast<int>(rot_dim),
        q_out, out_stride0, out_stride1, q_scales_out, scale_stride0, scale_stride1, weights, weights_stride, weights_dtype,
        weights_out, weights_out_stride, softmax_scale, head_scale, num_tokens, static_cast<int>(num_heads),
        static_cast<int>(head_dim), use_fp4 ? 1 : 0, static_cast<cudaStream_t>(cuda_stream)));
}

int dsv4_device_error(int32_t* value_host) {
    if (!value_host) return DSV4_ERR_NULL_POINTER;
    int v = 0;
    const cudaError_t err = read_device_error(&v);
    *value_host = v;
    return static_cast<int>(err);
}

int dsv4_set_variant(int variant) {
    if (variant < DSV4_VARIANT_AUTO || variant > DSV4_VARIANT_BULK) return DSV4_ERR_BAD_VARIANT;
    const int previous = current_variant();
    g_variant.store(variant, std::memory_order_relaxed);
    return previous;
}

int dsv4_get_variant(void) { return current_variant(); }

int dsv4_set_pdl(int mode) {
    const int previous = current_pdl();
    g_pdl.store(mode < 0 || mode > 2 ? 2 : mode, std::memory_order_relaxed);
    return previous;
}

int64_t dsv4_set_bulk_wait_cycles(int64_t cycles) {
    const long long previous = g_bulk_wait_cycles.load(std::memory_order_relaxed);
    if (cycles > 0) g_bulk_wait_cycles.store(cycles > 2000000000LL ? 2000000000LL : cycles, std::memory_order_relaxed);
    return previous;
}

int dsv4_bulk_wait_selftest(void* q, const void* kv, void* k_cache, const int64_t* slot_mapping, const int64_t* position_ids,
                            const float* cos_sin_cache, float eps, int64_t num_tokens, int64_t num_heads,
                            int64_t num_tokens_insert, int64_t cache_block_size, int64_t kv_block_stride_bytes,
                            int64_t short_tile, void* cuda_stream) {
    const int rc = validate(q, kv, k_cache, slot_mapping, position_ids, cos_sin_cache, num_tokens, num_heads,
                            num_tokens_insert, cache_block_size, kv_block_stride_bytes);
    if (rc != DSV4_OK || num_tokens == 0) return rc;
    if (short_tile < 0 || short_tile >= 0xffffffffLL) return DSV4_ERR_BAD_SIZE;
    PrologueParams p = make_params(q, kv, k_cache, slot_mapping, position_ids, cos_sin_cache, eps, num_tokens, num_heads,
                                   num_tokens_insert, cache_block_size, kv_block_stride_bytes);
    p.short_tile = static_cast<uint32_t>(short_tile);
    return static_cast<int>(launch_prologue_bulk(p, static_cast<cudaStream_t>(cuda_stream)));
}

int dsv4_set_table_staging(int mode) {
    const int previous = current_table_staging();
    g_table_staging.store(mode < -1 || mode > 1 ? -1 : mode, std::memory_order_relaxed);
    return previous;
}

int64_t dsv4_launch_count(void) { return g_launches.load(std::memory_order_relaxed); }

const char* dsv4_error_string(int code) {
    switch (code) {
        case DSV4_OK: return "success";
        case DSV4_ERR_NULL_POINTER: return "a required pointer is NULL";
        case DSV4_ERR_BAD_SIZE: return "bad size (negative, num_tokens_insert > num_tokens, or cache block too small)";
        case DSV4_ERR_MISALIGNED: return "a pointer or stride is not aligned as this entry point requires (see include/dsv4_prologue.h)";
        case DSV4_ERR_BAD_VARIANT: return "unknown kernel variant";
        case DSV4_ERR_TOO_LARGE: return "size exceeds what this entry point supports";
        default: return code > 0 ? cudaGetErrorString(static_cast<cudaError_t>(code)) : "unknown dsv4 error";
    }
}

const char* dsv4_version(void) { return "dsv4-prologue 0.1 sm_100a"; }

}  // extern "C"
