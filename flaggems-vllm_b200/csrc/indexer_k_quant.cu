// indexer_k_quant_and_cache: FP8 quantisation of the sparse-indexer keys k [N, head_dim] (bf16 or fp16)
// into a paged cache through slot_mapping - the sibling of the prologue's KV insert.
// Reference: src/flaggems_vllm/ops/indexer_k_quant_and_cache.py:44-132 and its torch statement
// tests/test_indexer_k_quant_and_cache.py:99-143:
//   per group of quant_block_size values: scale = max(amax, 1e-4) / 448 (made a power of two, rounded
//   up, for scale_fmt "ue8m0"); value = e4m3(x / scale); scale stored as fp32.
// Cache block b (stride given): block_size*head_dim e4m3 bytes, then block_size*(head_dim/qbs) fp32 scales.
// One warp per token, 8 values per lane per pass of 256 values; a group is qbs/8 adjacent lanes.
#include <cuda_fp16.h>

#include "dsv4_common.cuh"

namespace dsv4 {
namespace {

struct IndexerParams {
    const uint8_t* k;  // [N, head_dim] 16-bit floats, row stride in elements
    int64_t k_stride;
    uint8_t* cache;
    int64_t block_stride;  // bytes
    const int64_t* slot_mapping;
    int64_t num_tokens, block_size;
    int32_t head_dim, quant_block, num_quant_blocks;
    int32_t ue8m0, vec_ok;
    int32_t bs_shift;  // log2(block_size) or -1
};

template <bool FP16>
__device__ __forceinline__ void unpack8_any(const uint4& v, float (&x)[8]) {
    if (FP16) {
        const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w[i]));
            x[2 * i] = f.x, x[2 * i + 1] = f.y;
        }
    } else {
        unpack8(v, x);
    }
}

__device__ __forceinline__ float group_scale(float amax, bool ue8m0) {
    float s = __fdiv_rn(fmaxf(amax, 1e-4f), 448.0f);
    if (ue8m0) {  // 2^ceil(log2 s) from the bit pattern: exponent field, plus one if any mantissa bit is set
        const uint32_t u = __float_as_uint(s);
        s = __uint_as_float((((u >> 23) & 0xffu) + ((u & 0x7fffffu) ? 1u : 0u)) << 23);
    }
    return s;
}

template <int WARPS, bool FP16>
__global__ void __launch_bounds__(WARPS * 32) indexer_k_quant_kernel(const IndexerParams p) {
    const int lane = threadIdx.x & 31;
    const int64_t t = static_cast<int64_t>(blockIdx.x) * WARPS + (threadIdx.x >> 5);
    if (t >= p.num_tokens) return;
    const int64_t slot = p.slot_mapping[t];
    if (slot < 0) return;
    const int64_t block = slot / p.block_size, in_block = slot - block * p.block_size;
    uint8_t* base = p.cache + block * p.block_stride;
    uint8_t* values = base + in_block * p.head_dim;
    float* scales = reinterpret_cast<float*>(base + p.block_size * p.head_dim) + in_block * p.num_quant_blocks;
    const uint8_t* row = p.k + t * p.k_stride * 2;
    if (p.vec_ok) {
        const int group_lanes = p.quant_block >> 3;  // power of two, 1..32
        for (int e0 = 0; e0 < p.head_dim; e0 += 256) {
            const int e = e0 + 8 * lane;
            float x[8];
            uint4 v = make_uint4(0u, 0u, 0u, 0u);
            if (e < p.head_dim) v = ld_stream16(row + 2 * e);
            unpack8_any<FP16>(v, x);
            float amax = 0.0f;
#pragma unroll
            for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(x[i]));
            for (int m = 1; m < group_lanes; m <<= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, m));
            const float s = group_scale(amax, p.ue8m0 != 0);
            if (e < p.head_dim) {
#pragma unroll
                for (int i = 0; i < 8; ++i) x[i] = __fdiv_rn(x[i], s);
                st_global8(values + e, make_uint2(pack_e4m3x4(x[0], x[1], x[2], x[3]), pack_e4m3x4(x[4], x[5], x[6], x[7])));
                if ((lane & (group_lanes - 1)) == 0) scales[e / p.quant_block] = s;
            }
        }
    } else {
        // any quant_block / alignment: one group at a time, scalar accesses
        const uint16_t* row16 = reinterpret_cast<const uint16_t*>(row);
        for (int gq = 0; gq < p.num_quant_blocks; ++gq) {
            float amax = 0.0f;
            for (int i = lane; i < p.quant_block; i += 32) {
                const uint16_t h = row16[gq * p.quant_block + i];
                amax = fmaxf(amax, fabsf(FP16 ? __half2float(__ushort_as_half(h)) : bf16_lo(h)));
            }
#pragma unroll
            for (int m = 16; m > 0; m >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, m));
            const float s = group_scale(amax, p.ue8m0 != 0);
            for (int i = lane; i < p.quant_block; i += 32) {
                const uint16_t h = row16[gq * p.quant_block + i];
                const float q = __fdiv_rn(FP16 ? __half2float(__ushort_as_half(h)) : bf16_lo(h), s);
                values[gq * p.quant_block + i] = static_cast<uint8_t>(pack_e4m3x4(q, 0.f, 0.f, 0.f) & 0xffu);
            }
            if (lane == 0) scales[gq] = s;
        }
    }
}

// Fast shape for head_dim 64 / 128 / 256: a token is G = head_dim/8 lanes of 16 bytes, so one warp instruction
// moves 32/G tokens, and U passes are loaded (slot and row) before any is used.
template <int WARPS, int G, int U, bool FP16>
__global__ void __launch_bounds__(WARPS * 32) indexer_k_quant_rows_kernel(const IndexerParams p) {
    constexpr int TOKENS = 32 / G;
    const int lane = threadIdx.x & 31, sub = lane % G, which = lane / G;
    const int64_t base = (static_cast<int64_t>(blockIdx.x) * WARPS + (threadIdx.x >> 5)) * (U * TOKENS) + which;
    uint4 raw[U];
    int64_t slot[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
        const int64_t t = base + u * TOKENS;
        slot[u] = t < p.num_tokens ? p.slot_mapping[t] : -1;
        raw[u] = make_uint4(0u, 0u, 0u, 0u);
        if (slot[u] >= 0) raw[u] = ld_stream16(p.k + (t * p.k_stride + 8 * sub) * 2);
    }
    const int group_lanes = p.quant_block >> 3;  // power of two <= G
#pragma unroll
    for (int u = 0; u < U; ++u) {
        float x[8];
        unpack8_any<FP16>(raw[u], x);
        float amax = 0.0f;
#pragma unroll
        for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(x[i]));
        for (int m = 1; m < group_lanes; m <<= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, m));
        if (slot[u] < 0) continue;
        int64_t block, in_block;
        split_slot(slot[u], p.block_size, p.bs_shift, &block, &in_block);
        uint8_t* blk = p.cache + block * p.block_stride;
        float s;
        if (p.ue8m0) {
            const uint32_t code = ue8m0_code(amax);  // 2^ceil(log2(max(amax, 1e-4)/448)) without dividing
            s = __uint_as_float(code << 23);
            const float inv = __uint_as_float((254u - code) << 23);  // exact reciprocal of a power of two
#pragma unroll
            for (int i = 0; i < 8; ++i) x[i] = __fmul_rn(x[i], inv);
        } else {
            s = group_scale(amax, false);
#pragma unroll
            for (int i = 0; i < 8; ++i) x[i] = __fdiv_rn(x[i], s);
        }
        st_global8(blk + in_block * p.head_dim + 8 * sub, make_uint2(pack_e4m3x4(x[0], x[1], x[2], x[3]), pack_e4m3x4(x[4], x[5], x[6], x[7])));
        if ((sub & (group_lanes - 1)) == 0)
            reinterpret_cast<float*>(blk + p.block_size * p.head_dim)[in_block * p.num_quant_blocks + sub / group_lanes] = s;
    }
}

// The DeepSeek-V4 indexer shape (head_dim = quant_block = 128): 8 lanes per token, lane s keeps values [8s, 8s+8)
// and [64+8s, 64+8s+8), one scale per token; 4 tokens per warp instruction, U passes in flight.
#ifndef DSV4_INDEXER_K_CTAS
#define DSV4_INDEXER_K_CTAS 1
#endif
// UE8M0 (power-of-two scales): bf16 keys stay packed - group maximum and scaling on the bf16x2 words, as in quant8_pow2.
template <int WARPS, int U, bool FP16, bool UE8M0>
__global__ void __launch_bounds__(WARPS * 32, DSV4_INDEXER_K_CTAS) indexer_k_quant_128_kernel(const IndexerParams p) {
    const int lane = threadIdx.x & 31, sub = lane & 7, which = lane >> 3;
    const int64_t base = (static_cast<int64_t>(blockIdx.x) * WARPS + (threadIdx.x >> 5)) * (U * 4) + which;
    uint4 lo[U], hi[U];
    int64_t slot[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
        // the key row is fetched whether or not its slot turns out to be a skipped one (-1): the row load then does
        // not wait for the slot, and padding tokens are few
        const int64_t t = base + u * 4;
        slot[u] = -1;
        lo[u] = hi[u] = make_uint4(0u, 0u, 0u, 0u);
        if (t < p.num_tokens) {
            const uint8_t* row = p.k + (t * p.k_stride + 8 * sub) * 2;
            slot[u] = p.slot_mapping[t];
            lo[u] = ld_stream16(row);
            hi[u] = ld_stream16(row + 128);
        }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
        if (UE8M0 && !FP16) {
            uint32_t pk = max_abs_bf16x2(max_abs_bf16x2(max_abs_bf16x2(lo[u].x, lo[u].y), max_abs_bf16x2(lo[u].z, lo[u].w)),
                                         max_abs_bf16x2(max_abs_bf16x2(hi[u].x, hi[u].y), max_abs_bf16x2(hi[u].z, hi[u].w))) & 0x7fff7fffu;
#pragma unroll
            for (int m = 1; m < 8; m <<= 1) pk = max_bf16x2(pk, __shfl_xor_sync(0xffffffffu, pk, m));
            if (slot[u] < 0) continue;
            const uint32_t code = ue8m0_code(fmaxf(bf16_lo(pk), bf16_hi(pk)));
            int64_t block, in_block;
            split_slot(slot[u], p.block_size, p.bs_shift, &block, &in_block);
            uint8_t* blk = p.cache + block * p.block_stride;
            uint8_t* dst = blk + in_block * 128 + 8 * sub;
            st_global8(dst, quant8_pow2(lo[u], code));
            st_global8(dst + 64, quant8_pow2(hi[u], code));
            if (sub == 0) reinterpret_cast<float*>(blk + p.block_size * 128)[in_block] = __uint_as_float(code << 23);
            continue;
        }
        float x[8], y[8];
        unpack8_any<FP16>(lo[u], x);
        unpack8_any<FP16>(hi[u], y);
        float amax = 0.0f;
#pragma unroll
        for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fmaxf(fabsf(x[i]), fabsf(y[i])));
#pragma unroll
        for (int m = 1; m < 8; m <<= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, m));
        if (slot[u] < 0) continue;
        int64_t block, in_block;
        split_slot(slot[u], p.block_size, p.bs_shift, &block, &in_block);
        uint8_t* blk = p.cache + block * p.block_stride;
        uint8_t* dst = blk + in_block * 128 + 8 * sub;
        float s;
        if (UE8M0) {
            const uint32_t code = ue8m0_code(amax);
            s = __uint_as_float(code << 23);
            const float inv = __uint_as_float((254u - code) << 23);
#pragma unroll
            for (int i = 0; i < 8; ++i) x[i] = __fmul_rn(x[i], inv), y[i] = __fmul_rn(y[i], inv);
        } else {
            s = group_scale(amax, false);
#pragma unroll
            for (int i = 0; i < 8; ++i) x[i] = __fdiv_rn(x[i], s), y[i] = __fdiv_rn(y[i], s);
        }
        st_global8(dst, make_uint2(pack_e4m3x4(x[0], x[1], x[2], x[3]), pack_e4m3x4(x[4], x[5], x[6], x[7])));
        st_global8(dst + 64, make_uint2(pack_e4m3x4(y[0], y[1], y[2], y[3]), pack_e4m3x4(y[4], y[5], y[6], y[7])));
        if (sub == 0) reinterpret_cast<float*>(blk + p.block_size * 128)[in_block] = s;
    }
}

template <int G, bool FP16>
void launch_rows(const IndexerParams& p, cudaStream_t stream) {
    constexpr int WARPS = 4, U = 2, PER_CTA = WARPS * U * (32 / G);
    const unsigned grid = static_cast<unsigned>((p.num_tokens + PER_CTA - 1) / PER_CTA);
    indexer_k_quant_rows_kernel<WARPS, G, U, FP16><<<grid, WARPS * 32, 0, stream>>>(p);
}

}  // namespace

cudaError_t launch_indexer_k_quant(const void* k, int64_t k_stride, int is_fp16, void* cache, int64_t block_stride,
                                   const int64_t* slot_mapping, int64_t num_tokens, int64_t block_size, int head_dim,
                                   int quant_block, int ue8m0, cudaStream_t stream) {
    constexpr int WARPS = 4;
    if (num_tokens == 0) return cudaSuccess;
    IndexerParams p{};
    p.k = static_cast<const uint8_t*>(k), p.k_stride = k_stride, p.cache = static_cast<uint8_t*>(cache);
    p.block_stride = block_stride, p.slot_mapping = slot_mapping, p.num_tokens = num_tokens, p.block_size = block_size;
    p.bs_shift = pow2_shift(block_size);
    p.head_dim = head_dim, p.quant_block = quant_block, p.num_quant_blocks = head_dim / quant_block, p.ue8m0 = ue8m0;
    const bool pow2 = (quant_block & (quant_block - 1)) == 0;
    const auto addr = [](const void* q) { return reinterpret_cast<uintptr_t>(q); };
    p.vec_ok = pow2 && quant_block >= 8 && quant_block <= 256 && (addr(k) & 15u) == 0 && k_stride % 8 == 0 &&
               (addr(cache) & 7u) == 0 && block_stride % 8 == 0 && head_dim % 8 == 0 && (block_size * head_dim) % 4 == 0;
    const int64_t grid = (num_tokens + WARPS - 1) / WARPS;
    if (grid > 0x7fffffffLL) return cudaErrorInvalidConfiguration;
    if (p.vec_ok && head_dim == 128 && quant_block == 128) {
#ifndef DSV4_INDEXER_K_U
#define DSV4_INDEXER_K_U 2  // passes of 4 tokens a warp keeps in flight
#endif
        constexpr int W = 4, U = DSV4_INDEXER_K_U;
        const unsigned g128 = static_cast<unsigned>((num_tokens + W * U * 4 - 1) / (W * U * 4));
        if (is_fp16) ue8m0 ? indexer_k_quant_128_kernel<W, U, true, true><<<g128, W * 32, 0, stream>>>(p)
                           : indexer_k_quant_128_kernel<W, U, true, false><<<g128, W * 32, 0, stream>>>(p);
        else ue8m0 ? indexer_k_quant_128_kernel<W, U, false, true><<<g128, W * 32, 0, stream>>>(p)
                   : indexer_k_quant_128_kernel<W, U, false, false><<<g128, W * 32, 0, stream>>>(p);
        count_launch();
        return cudaGetLastError();
    }
    if (p.vec_ok && (head_dim == 64 || head_dim == 128 || head_dim == 256)) {
        if (head_dim == 64) is_fp16 ? launch_rows<8, true>(p, stream) : launch_rows<8, false>(p, stream);
        else if (head_dim == 128) is_fp16 ? launch_rows<16, true>(p, stream) : launch_rows<16, false>(p, stream);
        else is_fp16 ? launch_rows<32, true>(p, stream) : launch_rows<32, false>(p, stream);
        count_launch();
        return cudaGetLastError();
    }
    if (is_fp16) indexer_k_quant_kernel<WARPS, true><<<static_cast<unsigned>(grid), WARPS * 32, 0, stream>>>(p);
    else indexer_k_quant_kernel<WARPS, false><<<static_cast<unsigned>(grid), WARPS * 32, 0, stream>>>(p);
    count_launch();
    return cudaGetLastError();
}

}  // namespace dsv4
