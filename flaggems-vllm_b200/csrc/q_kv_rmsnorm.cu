// fused_q_kv_rmsnorm: the step before the prologue - weighted RMSNorm of the q low-rank
// activations [N, Q] and of the latent KV [N, KV] in one launch.
// Reference: src/flaggems_vllm/ops/deepseek_v4_attention_fused_q_kv_rmsnorm.py:24-103
//   y = (x * rsqrt(mean(x^2) + eps)) * w, fp32 arithmetic, bf16 in and out.
// One warp per row; a row of up to 2048 elements stays in registers between the reduction and
// the scaling (one read, one write per element); longer or unaligned rows take a two-pass
// scalar path.  Row 2t is the q row of token t, row 2t+1 its kv row.
#include <cuda_fp16.h>

#include "dsv4_common.cuh"

namespace dsv4 {
namespace {

struct NormRows {
    const uint8_t* in;
    uint8_t* out;
    const uint8_t* weight;
    int64_t in_stride, out_stride;  // elements
    int32_t size;
    int32_t vec_ok;                 // 16-byte path usable for this tensor
};

constexpr int kMaxChunks = 8;  // at most 8 16-byte chunks per lane are held in registers: 8 * 32 * 8 = 2048 elements

__device__ __forceinline__ float inv_rms_of(float sum, int size, float eps) {
    const float v = __fadd_rn(__fdiv_rn(sum, static_cast<float>(size)), eps);
    const float r0 = rsqrtf(v);
    return fmaf(r0, fmaf(-0.5f * v * r0, r0, 0.5f), r0);
}

// CH = chunks per lane the launch needs (2, 4, 6 or 8): fewer live registers for the common 1536 / 512 rows.
template <int WARPS, int CH>
__global__ void __launch_bounds__(WARPS * 32, CH <= 2 ? 16 : (CH <= 6 ? 8 : 6)) q_kv_rmsnorm_kernel(const NormRows q, const NormRows kv, int64_t num_tokens,
                                                                 float eps) {
    const int lane = threadIdx.x & 31;
    const int64_t r = static_cast<int64_t>(blockIdx.x) * WARPS + (threadIdx.x >> 5);
    if (r >= 2 * num_tokens) return;
    const bool is_q = (r & 1) == 0;  // rows alternate q, kv, q, kv ... so long and short rows mix in every CTA
    const NormRows& t = is_q ? q : kv;
    const int64_t token = r >> 1;
    const uint8_t* in = t.in + token * t.in_stride * 2;
    uint8_t* out = t.out + token * t.out_stride * 2;
    const int size = t.size;
    if (t.vec_ok) {
        const int chunks = size >> 3;
        uint4 x[CH];
        float acc = 0.0f;
#pragma unroll
        for (int j = 0; j < CH; ++j) {
            const int c = lane + 32 * j;
            x[j] = make_uint4(0u, 0u, 0u, 0u);
            if (c < chunks) x[j] = ld_stream16(in + 16 * c);
        }
#pragma unroll
        for (int j = 0; j < CH; ++j) {
            float f[8];
            unpack8(x[j], f);
#pragma unroll
            for (int i = 0; i < 8; ++i) acc = fmaf(f[i], f[i], acc);
        }
#pragma unroll
        for (int m = 16; m > 0; m >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, m);
        const float rr = inv_rms_of(acc, size, eps);
#pragma unroll
        for (int j = 0; j < CH; ++j) {
            const int c = lane + 32 * j;
            if (c < chunks) {
                float f[8], w[8];
                unpack8(x[j], f);
                unpack8(__ldg(reinterpret_cast<const uint4*>(t.weight + 16 * c)), w);
#pragma unroll
                for (int i = 0; i < 8; ++i) f[i] = __fmul_rn(__fmul_rn(f[i], rr), w[i]);
                st_stream16(out + 16 * c, pack8(f));
            }
        }
    } else {
        const uint16_t* in16 = reinterpret_cast<const uint16_t*>(in);
        const uint16_t* w16 = reinterpret_cast<const uint16_t*>(t.weight);
        uint16_t* out16 = reinterpret_cast<uint16_t*>(out);
        float acc = 0.0f;
        for (int i = lane; i < size; i += 32) {
            const float f = bf16_lo(in16[i]);
            acc = fmaf(f, f, acc);
        }
#pragma unroll
        for (int m = 16; m > 0; m >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, m);
        const float rr = inv_rms_of(acc, size, eps);
        for (int i = lane; i < size; i += 32) {
            const float y = __fmul_rn(__fmul_rn(bf16_lo(in16[i]), rr), bf16_lo(w16[i]));
            out16[i] = static_cast<uint16_t>(pack_bf16x2(y, 0.0f) & 0xffffu);
        }
    }
}

// Any of bf16 (0), fp16 (1), fp32 (2) for the rows and, independently, for the weights: the reference kernel is
// generic over the element types (it loads everything as fp32 and stores in the output's type).  One warp per row,
// two passes over the row, element by element.  The DeepSeek-V4 layer passes bf16 everywhere and takes the kernel above.
struct AnyRows {
    const uint8_t* in;
    uint8_t* out;
    const uint8_t* weight;
    int64_t in_stride, out_stride;  // elements
    int32_t size, dtype, weight_dtype;
};

__device__ __forceinline__ float load_any(const uint8_t* base, int64_t i, int dtype) {
    if (dtype == 2) return reinterpret_cast<const float*>(base)[i];
    const uint16_t h = reinterpret_cast<const uint16_t*>(base)[i];
    return dtype == 0 ? bf16_lo(h) : __half2float(__ushort_as_half(h));
}

__device__ __forceinline__ void store_any(uint8_t* base, int64_t i, int dtype, float v) {
    if (dtype == 2) reinterpret_cast<float*>(base)[i] = v;
    else if (dtype == 0) reinterpret_cast<uint16_t*>(base)[i] = static_cast<uint16_t>(pack_bf16x2(v, 0.0f) & 0xffffu);
    else reinterpret_cast<uint16_t*>(base)[i] = __half_as_ushort(__float2half_rn(v));
}

template <int WARPS>
__global__ void __launch_bounds__(WARPS * 32) q_kv_rmsnorm_any_kernel(const AnyRows q, const AnyRows kv, int64_t num_tokens, float eps) {
    const int lane = threadIdx.x & 31;
    const int64_t r = static_cast<int64_t>(blockIdx.x) * WARPS + (threadIdx.x >> 5);
    if (r >= 2 * num_tokens) return;
    const AnyRows& t = (r & 1) == 0 ? q : kv;
    const int64_t token = r >> 1;
    const int esize = t.dtype == 2 ? 4 : 2;
    const uint8_t* in = t.in + token * t.in_stride * esize;
    uint8_t* out = t.out + token * t.out_stride * esize;
    float acc = 0.0f;
    for (int i = lane; i < t.size; i += 32) {
        const float f = load_any(in, i, t.dtype);
        acc = fmaf(f, f, acc);
    }
#pragma unroll
    for (int m = 16; m > 0; m >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, m);
    const float rr = inv_rms_of(acc, t.size, eps);
    for (int i = lane; i < t.size; i += 32)
        store_any(out, i, t.dtype, __fmul_rn(__fmul_rn(load_any(in, i, t.dtype), rr), load_any(t.weight, i, t.weight_dtype)));
}

bool vec_ok(const void* in, const void* out, const void* w, int64_t in_stride, int64_t out_stride, int64_t size) {
    const auto a = [](const void* p) { return reinterpret_cast<uintptr_t>(p) & 15u; };
    return a(in) == 0 && a(out) == 0 && a(w) == 0 && in_stride % 8 == 0 && out_stride % 8 == 0 && size % 8 == 0 &&
           size <= kMaxChunks * 256;
}

}  // namespace

cudaError_t launch_q_kv_rmsnorm(const void* q, void* q_out, const void* q_weight, int64_t q_in_stride, int64_t q_out_stride,
                                int64_t q_size, const void* kv, void* kv_out, const void* kv_weight, int64_t kv_in_stride,
                                int64_t kv_out_stride, int64_t kv_size, int64_t num_tokens, float eps, cudaStream_t stream) {
    constexpr int WARPS = 4;
    if (num_tokens == 0) return cudaSuccess;
    NormRows a{static_cast<const uint8_t*>(q), static_cast<uint8_t*>(q_out), static_cast<const uint8_t*>(q_weight),
               q_in_stride, q_out_stride, static_cast<int32_t>(q_size),
               vec_ok(q, q_out, q_weight, q_in_stride, q_out_stride, q_size) ? 1 : 0};
    NormRows b{static_cast<const uint8_t*>(kv), static_cast<uint8_t*>(kv_out), static_cast<const uint8_t*>(kv_weight),
               kv_in_stride, kv_out_stride, static_cast<int32_t>(kv_size),
               vec_ok(kv, kv_out, kv_weight, kv_in_stride, kv_out_stride, kv_size) ? 1 : 0};
    const int64_t grid = (2 * num_tokens + WARPS - 1) / WARPS;
    if (grid > 0x7fffffffLL) return cudaErrorInvalidConfiguration;
    const int64_t longest = (a.vec_ok ? q_size : 0) > (b.vec_ok ? kv_size : 0) ? (a.vec_ok ? q_size : 0) : (b.vec_ok ? kv_size : 0);
    const unsigned g = static_cast<unsigned>(grid);
    if (longest <= 512) q_kv_rmsnorm_kernel<WARPS, 2><<<g, WARPS * 32, 0, stream>>>(a, b, num_tokens, eps);
    else if (longest <= 1024) q_kv_rmsnorm_kernel<WARPS, 4><<<g, WARPS * 32, 0, stream>>>(a, b, num_tokens, eps);
    else if (longest <= 1536) q_kv_rmsnorm_kernel<WARPS, 6><<<g, WARPS * 32, 0, stream>>>(a, b, num_tokens, eps);
    else q_kv_rmsnorm_kernel<WARPS, 8><<<g, WARPS * 32, 0, stream>>>(a, b, num_tokens, eps);
    count_launch();
    return cudaGetLastError();
}

cudaError_t launch_q_kv_rmsnorm_any(const void* q, void* q_out, const void* q_weight, int64_t q_in_stride, int64_t q_out_stride,
                                    int64_t q_size, int q_dtype, int q_weight_dtype, const void* kv, void* kv_out,
                                    const void* kv_weight, int64_t kv_in_stride, int64_t kv_out_stride, int64_t kv_size,
                                    int kv_dtype, int kv_weight_dtype, int64_t num_tokens, float eps, cudaStream_t stream) {
    constexpr int WARPS = 4;
    if (num_tokens == 0) return cudaSuccess;
    const AnyRows a{static_cast<const uint8_t*>(q), static_cast<uint8_t*>(q_out), static_cast<const uint8_t*>(q_weight),
                    q_in_stride, q_out_stride, static_cast<int32_t>(q_size), q_dtype, q_weight_dtype};
    const AnyRows b{static_cast<const uint8_t*>(kv), static_cast<uint8_t*>(kv_out), static_cast<const uint8_t*>(kv_weight),
                    kv_in_stride, kv_out_stride, static_cast<int32_t>(kv_size), kv_dtype, kv_weight_dtype};
    const int64_t grid = (2 * num_tokens + WARPS - 1) / WARPS;
    if (grid > 0x7fffffffLL) return cudaErrorInvalidConfiguration;
    q_kv_rmsnorm_any_kernel<WARPS><<<static_cast<unsigned>(grid), WARPS * 32, 0, stream>>>(a, b, num_tokens, eps);
    count_launch();
    return cudaGetLastError();
}

}  // namespace dsv4
