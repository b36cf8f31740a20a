// Reader of the cache rows the prologue writes: one warp per slot turns the 448 e4m3
// bytes + 7 UE8M0 codes back into bf16 and copies the 64 cached bf16 RoPE values.
// Per-token arithmetic of the reference's dequantize_and_gather_k_cache
// (src/flaggems_vllm/ops/deepseek_v4_attention_dequantize_and_gather_k_cache.py:86-120):
// value = e4m3 * 2^(code - 127), rounded to bf16.
#include "dsv4_common.cuh"

namespace dsv4 {
namespace {

// 2^(code-127) for a stored UE8M0 byte (0 -> 2^-127 as a subnormal, 255 -> +inf, as exp2f gives).
__device__ __forceinline__ float ue8m0_to_float(uint32_t code) {
    if (code == 0u) return __uint_as_float(0x00400000u);
    if (code == 255u) return __uint_as_float(0x7f800000u);
    return __uint_as_float(code << 23);
}

__device__ __forceinline__ uint4 dequant8(uint2 bytes, float scale) {
    const float2 p0 = unpack_e4m3x2(static_cast<uint16_t>(bytes.x & 0xffffu));
    const float2 p1 = unpack_e4m3x2(static_cast<uint16_t>(bytes.x >> 16));
    const float2 p2 = unpack_e4m3x2(static_cast<uint16_t>(bytes.y & 0xffffu));
    const float2 p3 = unpack_e4m3x2(static_cast<uint16_t>(bytes.y >> 16));
    return make_uint4(pack_bf16x2(__fmul_rn(p0.x, scale), __fmul_rn(p0.y, scale)),
                      pack_bf16x2(__fmul_rn(p1.x, scale), __fmul_rn(p1.y, scale)),
                      pack_bf16x2(__fmul_rn(p2.x, scale), __fmul_rn(p2.y, scale)),
                      pack_bf16x2(__fmul_rn(p3.x, scale), __fmul_rn(p3.y, scale)));
}

template <typename T>
__device__ __forceinline__ T load_bytes(const uint8_t* p, bool aligned) {
    if (aligned) return *reinterpret_cast<const T*>(p);
    T v;
    uint8_t* d = reinterpret_cast<uint8_t*>(&v);
#pragma unroll
    for (int i = 0; i < static_cast<int>(sizeof(T)); ++i) d[i] = p[i];
    return v;
}

template <int WARPS>
__global__ void __launch_bounds__(WARPS * 32)
gather_dequant_kernel(const uint8_t* __restrict__ k_cache, const int64_t* __restrict__ slots, int64_t num_slots,
                      uint8_t* __restrict__ out, int64_t out_row_bytes, int64_t block_size, int64_t block_stride,
                      int aligned16) {
    const int lane = threadIdx.x & 31;
    const int64_t i = static_cast<int64_t>(blockIdx.x) * WARPS + (threadIdx.x >> 5);
    if (i >= num_slots) return;
    uint8_t* row = out + i * out_row_bytes;
    const int64_t slot = slots[i];
    if (slot < 0) {
        const uint4 z = make_uint4(0u, 0u, 0u, 0u);
        *reinterpret_cast<uint4*>(row + 16 * lane) = z;
        *reinterpret_cast<uint4*>(row + 512 + 16 * lane) = z;
        return;
    }
    const int64_t block = slot / block_size, in_block = slot - block * block_size;
    const uint8_t* base = k_cache + block * block_stride;
    const uint8_t* data = base + in_block * kTokenDataBytes;
    const uint8_t* scales = base + block_size * kTokenDataBytes + in_block * kScaleBytes;
    const bool al = aligned16 != 0;
    const uint2 codes = load_bytes<uint2>(scales, al);
    const int ga = lane >> 3, gb = 4 + (lane >> 3);  // quant group of register A / B of this lane
    const float scale_a = ue8m0_to_float((codes.x >> (8 * ga)) & 0xffu);
    *reinterpret_cast<uint4*>(row + 16 * lane) = dequant8(load_bytes<uint2>(data + 8 * lane, al), scale_a);
    uint4 b;
    if (lane >= kFirstRopeLane) {
        b = load_bytes<uint4>(data + kNopeDim + 16 * (lane - kFirstRopeLane), al);
    } else {
        const float scale_b = ue8m0_to_float((codes.y >> (8 * (gb - 4))) & 0xffu);
        b = dequant8(load_bytes<uint2>(data + 256 + 8 * lane, al), scale_b);
    }
    *reinterpret_cast<uint4*>(row + 512 + 16 * lane) = b;
}

// ---- request / block-table form (the reference operator's own addressing) -------------------------
//
// out[r, offset + i, :] = token at position seq_len[r] - gather_len[r] + i of request r, found through
// block_table[r, pos / block_size].  grid = (CTAs per request, requests); the warps of a request stride
// over its gathered positions.  FAST = DeepSeek-V4 layout (448 e4m3 + 64 bf16, 8 scale bytes) with
// 16-byte aligned rows on both sides; otherwise any nope/rope/scale_slots with scalar accesses.
struct GatherParams {
    uint8_t* out;            // bf16, element strides below, unit stride in the last dimension
    int64_t out_stride0, out_stride1;
    const uint8_t* k_cache;
    const void* seq_lens;
    const void* gather_lens;  // may be null: gather the whole sequence
    const void* block_table;
    int64_t max_blocks_per_seq;
    int64_t block_size, block_stride;
    int64_t offset;
    int32_t nope_dim, rope_dim, scale_slots;
    int32_t index64;          // 1: seq_lens / gather_lens / block_table are int64, 0: int32
    int32_t bs_shift;         // log2(block_size) or -1
};

__device__ __forceinline__ int64_t load_index(const void* p, int64_t i, int is64) {
    return is64 ? static_cast<const int64_t*>(p)[i] : static_cast<int64_t>(static_cast<const int32_t*>(p)[i]);
}

template <int WARPS, bool FAST>
__global__ void __launch_bounds__(WARPS * 32) gather_dequant_requests_kernel(const GatherParams g) {
    const int lane = threadIdx.x & 31;
    const int64_t req = blockIdx.y;
    const int64_t seq_len = load_index(g.seq_lens, req, g.index64);
    const int64_t gather_len = g.gather_lens ? load_index(g.gather_lens, req, g.index64) : seq_len;
    const int64_t start = seq_len - gather_len;
    const int64_t token_data = g.nope_dim + 2 * g.rope_dim;
    const int64_t warps_per_req = static_cast<int64_t>(gridDim.x) * WARPS;
    const int64_t first = static_cast<int64_t>(blockIdx.x) * WARPS + (threadIdx.x >> 5);
    if (FAST) {
        // two tokens per warp and iteration: both block-table lookups, then all cache reads, are in flight
        // together before anything is converted
        constexpr int U = 2;
        for (int64_t i0 = first; i0 < gather_len; i0 += U * warps_per_req) {
            const uint8_t* data[U];
            const uint8_t* scales[U];
            int64_t block[U];
            bool live[U];
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const int64_t i = i0 + u * warps_per_req;
                live[u] = i < gather_len;
                const int64_t pos = start + (live[u] ? i : i0);
                const int64_t block_in_seq = g.bs_shift >= 0 ? pos >> g.bs_shift : pos / g.block_size;
                block[u] = load_index(g.block_table, req * g.max_blocks_per_seq + block_in_seq, g.index64);
            }
            uint2 codes[U], qa[U];
            uint4 qb[U];
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const int64_t pos = start + (live[u] ? i0 + u * warps_per_req : i0);
                const int64_t in_block = g.bs_shift >= 0 ? pos & (g.block_size - 1) : pos % g.block_size;
                const uint8_t* base = g.k_cache + block[u] * g.block_stride;
                data[u] = base + in_block * kTokenDataBytes;
                scales[u] = base + g.block_size * kTokenDataBytes + in_block * kScaleBytes;
                codes[u] = *reinterpret_cast<const uint2*>(scales[u]);
                qa[u] = *reinterpret_cast<const uint2*>(data[u] + 8 * lane);
                if (lane >= kFirstRopeLane) {
                    qb[u] = *reinterpret_cast<const uint4*>(data[u] + kNopeDim + 16 * (lane - kFirstRopeLane));
                } else {
                    const uint2 t = *reinterpret_cast<const uint2*>(data[u] + 256 + 8 * lane);
                    qb[u] = make_uint4(t.x, t.y, 0u, 0u);
                }
            }
#pragma unroll
            for (int u = 0; u < U; ++u) {
                if (!live[u]) continue;
                const int64_t i = i0 + u * warps_per_req;
                uint8_t* row = g.out + (req * g.out_stride0 + (g.offset + i) * g.out_stride1) * 2;
                const float scale_a = ue8m0_to_float((codes[u].x >> (8 * (lane >> 3))) & 0xffu);
                *reinterpret_cast<uint4*>(row + 16 * lane) = dequant8(qa[u], scale_a);
                uint4 b = qb[u];
                if (lane < kFirstRopeLane) {
                    const float scale_b = ue8m0_to_float((codes[u].y >> (8 * (lane >> 3))) & 0xffu);
                    b = dequant8(make_uint2(qb[u].x, qb[u].y), scale_b);
                }
                *reinterpret_cast<uint4*>(row + 512 + 16 * lane) = b;
            }
        }
    } else {
        for (int64_t i = first; i < gather_len; i += warps_per_req) {
            const int64_t pos = start + i;
            const int64_t block_in_seq = pos / g.block_size, in_block = pos - block_in_seq * g.block_size;
            const int64_t block = load_index(g.block_table, req * g.max_blocks_per_seq + block_in_seq, g.index64);
            const uint8_t* base = g.k_cache + block * g.block_stride;
            const uint8_t* data = base + in_block * token_data;
            const uint8_t* scales = base + g.block_size * token_data + in_block * g.scale_slots;
            uint8_t* row = g.out + (req * g.out_stride0 + (g.offset + i) * g.out_stride1) * 2;
            uint16_t* out16 = reinterpret_cast<uint16_t*>(row);
            for (int j = lane; j < g.nope_dim; j += 32) {
                const float scale = ue8m0_to_float(scales[j >> 6]);
                const float v = unpack_e4m3x2(static_cast<uint16_t>(data[j])).x;
                out16[j] = static_cast<uint16_t>(pack_bf16x2(__fmul_rn(v, scale), 0.0f) & 0xffffu);
            }
            for (int j = lane; j < g.rope_dim; j += 32)
                out16[g.nope_dim + j] = static_cast<uint16_t>(data[g.nope_dim + 2 * j]) |
                                        (static_cast<uint16_t>(data[g.nope_dim + 2 * j + 1]) << 8);
        }
    }
}

}  // namespace

cudaError_t launch_gather_dequant(const uint8_t* k_cache, const int64_t* slots, int64_t num_slots, uint8_t* out,
                                  int64_t out_row_stride, int64_t block_size, int64_t block_stride,
                                  cudaStream_t stream) {
    constexpr int WARPS = 8;
    if (num_slots == 0) return cudaSuccess;
    const int64_t grid = (num_slots + WARPS - 1) / WARPS;
    if (grid > 0x7fffffffLL) return cudaErrorInvalidConfiguration;
    const int aligned16 = ((reinterpret_cast<uintptr_t>(k_cache) | static_cast<uintptr_t>(block_stride)) & 15u) == 0;
    gather_dequant_kernel<WARPS><<<static_cast<unsigned>(grid), WARPS * 32, 0, stream>>>(
        k_cache, slots, num_slots, out, out_row_stride * 2, block_size, block_stride, aligned16);
    count_launch();
    return cudaGetLastError();
}

cudaError_t launch_gather_dequant_requests(uint8_t* out, int64_t out_stride0, int64_t out_stride1, const uint8_t* k_cache,
                                           const void* seq_lens, const void* gather_lens, const void* block_table,
                                           int64_t num_reqs, int64_t max_blocks_per_seq, int64_t block_size,
                                           int64_t block_stride, int64_t offset, int nope_dim, int rope_dim, int scale_slots,
                                           int index64, int64_t tokens_hint, cudaStream_t stream) {
    constexpr int WARPS = 8;
    if (num_reqs == 0) return cudaSuccess;
    if (num_reqs > 65535) return cudaErrorInvalidConfiguration;
    GatherParams g{};
    g.out = out, g.out_stride0 = out_stride0, g.out_stride1 = out_stride1, g.k_cache = k_cache;
    g.seq_lens = seq_lens, g.gather_lens = gather_lens, g.block_table = block_table;
    g.max_blocks_per_seq = max_blocks_per_seq, g.block_size = block_size, g.block_stride = block_stride, g.offset = offset;
    g.nope_dim = nope_dim, g.rope_dim = rope_dim, g.scale_slots = scale_slots, g.index64 = index64;
    g.bs_shift = pow2_shift(block_size);
    // gather lengths live on the device; size the grid from the room the output has per request
    int64_t ctas = (tokens_hint + WARPS - 1) / WARPS;
    if (ctas < 1) ctas = 1;
    if (ctas > 256) ctas = 256;
    const auto addr = [](const void* p) { return reinterpret_cast<uintptr_t>(p); };
    const bool fast = nope_dim == kNopeDim && rope_dim == kRopeDim && scale_slots == kScaleBytes &&
                      ((addr(k_cache) | static_cast<uintptr_t>(block_stride)) & 15u) == 0 && (addr(out) & 15u) == 0 &&
                      out_stride0 % 8 == 0 && out_stride1 % 8 == 0 && (block_size * kTokenDataBytes) % 8 == 0;
    const dim3 grid(static_cast<unsigned>(ctas), static_cast<unsigned>(num_reqs));
    if (fast) gather_dequant_requests_kernel<WARPS, true><<<grid, WARPS * 32, 0, stream>>>(g);
    else gather_dequant_requests_kernel<WARPS, false><<<grid, WARPS * 32, 0, stream>>>(g);
    count_launch();
    return cudaGetLastError();
}

}  // namespace dsv4
