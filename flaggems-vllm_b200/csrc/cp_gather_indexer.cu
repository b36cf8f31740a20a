// cp_gather_indexer_k_quant_cache: the reader of the sparse-indexer key cache that indexer_k_quant_and_cache
// writes.  Output token t belongs to the request b with cu_seqlen[b] <= t < cu_seqlen[b+1]; its bytes are copied
// from block block_table[b, (t - cu_seqlen[b]) / block_size], position (t - cu_seqlen[b]) % block_size:
// head_dim e4m3 bytes into k_out[t] and head_dim/quant_block fp32 scales into scale_out[t].  Tokens outside
// every request are left untouched, and so are tokens whose block-table entry is negative (an unused entry; the
// reference would read before the cache).
// Reference: src/flaggems_vllm/ops/cp_gather_indexer_k_quant_cache.py:24-190 and its torch statement
// tests/test_cp_gather_indexer_k_quant_cache.py:85-116.
// Cache block b (stride given): block_size*head_dim value bytes, then block_size*num_quant_blocks fp32 scales.
//
// HBM traffic: head_dim + 4*num_quant_blocks bytes read and the same written per token; nothing is computed.
#include "dsv4_common.cuh"

namespace dsv4 {
namespace {

struct CpGatherParams {
    const uint8_t* cache;
    int64_t block_stride;  // bytes
    uint8_t* k_out;
    int64_t k_out_stride;  // bytes
    uint8_t* scale_out;
    int64_t scale_out_stride;  // bytes
    const int32_t* block_table;
    int64_t block_table_stride;
    const int32_t* cu_seqlen;  // [batch + 1], non-decreasing
    int32_t batch, num_tokens;
    int32_t block_size, head_dim, num_quant_blocks;
    int32_t bs_shift;  // log2(block_size) or -1
    int32_t search_steps;
};

// Request of token t: the last b with cu_seqlen[b] <= t (bisection over [0, batch]), valid if t < cu_seqlen[b+1].
// Returns false for a token outside every request.
__device__ __forceinline__ bool locate(const CpGatherParams& p, int32_t t, int32_t* block, int32_t* in_block) {
    int32_t left = 0, right = p.batch + 1;
    for (int32_t s = 0; s < p.search_steps; ++s) {
        const int32_t mid = (left + right) >> 1;
        const bool before = mid <= p.batch && __ldg(p.cu_seqlen + mid) <= t;
        left = before ? mid + 1 : left;
        right = before ? right : mid;
    }
    const int32_t b = left - 1;
    if (b < 0 || b >= p.batch) return false;
    const int32_t start = __ldg(p.cu_seqlen + b);
    if (t < start || t >= __ldg(p.cu_seqlen + b + 1)) return false;
    const int32_t off = t - start;
    const int32_t idx = p.bs_shift >= 0 ? off >> p.bs_shift : off / p.block_size;
    *in_block = off - idx * p.block_size;
    *block = __ldg(p.block_table + static_cast<int64_t>(b) * p.block_table_stride + idx);
    return true;
}

// LANES adjacent lanes per token (16 value bytes each per pass), U tokens per lane group in flight, so a warp owns
// 32/LANES*U <= 32 consecutive tokens.  Lane i locates token i of the warp (one bisection per token, all of them
// side by side); the lane groups then fetch block and position of their tokens with shuffles.
template <int WARPS, int LANES, int U>
__global__ void __launch_bounds__(WARPS * 32) cp_gather_indexer_vec_kernel(const CpGatherParams p) {
    constexpr int kGroups = 32 / LANES;
    static_assert(kGroups * U <= 32, "a warp locates one token per lane");
    const int lane = threadIdx.x & 31;
    const int sub = lane % LANES;
    const int64_t warp_token0 = (static_cast<int64_t>(blockIdx.x) * WARPS + (threadIdx.x >> 5)) * (kGroups * U);
    const int64_t group0 = warp_token0 + lane / LANES;
    const int chunks = p.head_dim >> 4;
    int32_t my_block = -1, my_in_block = 0;
    if (lane < kGroups * U && warp_token0 + lane < p.num_tokens &&
        !locate(p, static_cast<int32_t>(warp_token0 + lane), &my_block, &my_in_block))
        my_block = -1;
    const uint8_t* src[U];
    const uint8_t* src_scale[U];
    bool ok[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
        const int from = lane / LANES + u * kGroups;
        const int32_t block = __shfl_sync(0xffffffffu, my_block, from);
        const int32_t in_block = __shfl_sync(0xffffffffu, my_in_block, from);
        ok[u] = block >= 0;
        const uint8_t* base = p.cache + static_cast<int64_t>(block) * p.block_stride;
        src[u] = base + static_cast<int64_t>(in_block) * p.head_dim;
        src_scale[u] = base + static_cast<int64_t>(p.block_size) * p.head_dim + static_cast<int64_t>(in_block) * p.num_quant_blocks * 4;
    }
    if (chunks <= LANES) {
        // one pass: all loads first, then all stores
        uint4 v[U];
        uint32_t s[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            v[u] = make_uint4(0u, 0u, 0u, 0u), s[u] = 0u;
            if (ok[u] && sub < chunks) v[u] = ld_stream16(src[u] + 16 * sub);
            if (ok[u] && sub < p.num_quant_blocks) s[u] = ld_stream4(src_scale[u] + 4 * sub);
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int64_t t = group0 + u * kGroups;
            if (ok[u] && sub < chunks) st_stream16(p.k_out + t * p.k_out_stride + 16 * sub, v[u]);
            if (ok[u] && sub < p.num_quant_blocks) st_stream4(p.scale_out + t * p.scale_out_stride + 4 * sub, s[u]);
        }
        if (p.num_quant_blocks <= LANES) return;
    } else {
#pragma unroll
        for (int u = 0; u < U; ++u) {
            if (!ok[u]) continue;
            const int64_t t = group0 + u * kGroups;
            for (int c = sub; c < chunks; c += LANES) st_stream16(p.k_out + t * p.k_out_stride + 16 * c, ld_stream16(src[u] + 16 * c));
        }
    }
    // scales beyond the first LANES (more quantisation groups than lanes per token)
#pragma unroll
    for (int u = 0; u < U; ++u) {
        if (!ok[u]) continue;
        const int64_t t = group0 + u * kGroups;
        for (int c = sub + (chunks <= LANES ? LANES : 0); c < p.num_quant_blocks; c += LANES)
            st_stream4(p.scale_out + t * p.scale_out_stride + 4 * c, ld_stream4(src_scale[u] + 4 * c));
    }
}

// Any head_dim and any alignment: one warp per token, byte by byte.
template <int WARPS>
__global__ void __launch_bounds__(WARPS * 32) cp_gather_indexer_bytes_kernel(const CpGatherParams p) {
    const int lane = threadIdx.x & 31;
    const int64_t t = static_cast<int64_t>(blockIdx.x) * WARPS + (threadIdx.x >> 5);
    if (t >= p.num_tokens) return;
    int32_t block = 0, in_block = 0;
    if (!locate(p, static_cast<int32_t>(t), &block, &in_block)) return;
    const uint8_t* base = p.cache + static_cast<int64_t>(block) * p.block_stride;
    const uint8_t* src = base + static_cast<int64_t>(in_block) * p.head_dim;
    const uint8_t* src_scale = base + static_cast<int64_t>(p.block_size) * p.head_dim + static_cast<int64_t>(in_block) * p.num_quant_blocks * 4;
    for (int i = lane; i < p.head_dim; i += 32) p.k_out[t * p.k_out_stride + i] = src[i];
    for (int i = lane; i < p.num_quant_blocks * 4; i += 32) p.scale_out[t * p.scale_out_stride + i] = src_scale[i];
}

}  // namespace

cudaError_t launch_cp_gather_indexer(const void* cache, int64_t block_stride, void* k_out, int64_t k_out_stride, void* scale_out,
                                     int64_t scale_out_stride, const int32_t* block_table, int64_t block_table_stride,
                                     const int32_t* cu_seqlen, int64_t batch, int64_t num_tokens, int64_t block_size, int head_dim,
                                     int num_quant_blocks, cudaStream_t stream) {
    if (num_tokens == 0 || batch == 0) return cudaSuccess;
    CpGatherParams p{};
    p.cache = static_cast<const uint8_t*>(cache), p.block_stride = block_stride;
    p.k_out = static_cast<uint8_t*>(k_out), p.k_out_stride = k_out_stride;
    p.scale_out = static_cast<uint8_t*>(scale_out), p.scale_out_stride = scale_out_stride;
    p.block_table = block_table, p.block_table_stride = block_table_stride, p.cu_seqlen = cu_seqlen;
    p.batch = static_cast<int32_t>(batch), p.num_tokens = static_cast<int32_t>(num_tokens);
    p.block_size = static_cast<int32_t>(block_size), p.head_dim = head_dim, p.num_quant_blocks = num_quant_blocks;
    p.bs_shift = pow2_shift(block_size);
    p.search_steps = 0;
    for (int64_t span = batch + 1; span > 0; span >>= 1) ++p.search_steps;  // bit length of batch + 1: every step at least halves [left, right), which starts at batch + 1 entries
    const auto addr = [](const void* q) { return reinterpret_cast<uintptr_t>(q); };
    const bool vec = head_dim % 16 == 0 && addr(cache) % 16 == 0 && block_stride % 16 == 0 && addr(k_out) % 16 == 0 &&
                     k_out_stride % 16 == 0 && addr(scale_out) % 4 == 0 && scale_out_stride % 4 == 0 &&
                     (block_size * static_cast<int64_t>(head_dim)) % 4 == 0;
    constexpr int WARPS = 4;
    if (!vec) {
        const int64_t grid = (num_tokens + WARPS - 1) / WARPS;
        if (grid > 0x7fffffffLL) return cudaErrorInvalidConfiguration;
        cp_gather_indexer_bytes_kernel<WARPS><<<static_cast<unsigned>(grid), WARPS * 32, 0, stream>>>(p);
    } else {
        constexpr int U = 4;
        const int chunks = head_dim / 16;
#define DSV4_CP_GATHER(LANES)                                                                                             \
    do {                                                                                                                  \
        const int64_t per_cta = static_cast<int64_t>(WARPS) * (32 / LANES) * U;                                           \
        const int64_t grid = (num_tokens + per_cta - 1) / per_cta;                                                        \
        if (grid > 0x7fffffffLL) return cudaErrorInvalidConfiguration;                                                    \
        cp_gather_indexer_vec_kernel<WARPS, LANES, U><<<static_cast<unsigned>(grid), WARPS * 32, 0, stream>>>(p);          \
    } while (0)
        if (chunks <= 4) DSV4_CP_GATHER(4);
        else if (chunks <= 8) DSV4_CP_GATHER(8);
        else if (chunks <= 16) DSV4_CP_GATHER(16);
        else DSV4_CP_GATHER(32);
#undef DSV4_CP_GATHER
    }
    count_launch();
    return cudaGetLastError();
}

}  // namespace dsv4
