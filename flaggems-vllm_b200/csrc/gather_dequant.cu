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

}  // namespace dsv4
