// fused_inv_rope_fp8_quant: the attention epilogue that mirrors the prologue - inverse GPT-J RoPE on
// the rotary tail of the attention output o [N, H, 512], then FP8 e4m3 quantisation in groups of 128
// with one scale per group (fp32 = amax/448, or a power of two packed as UE8M0 bytes).
// Reference: src/flaggems_vllm/ops/fused_inv_rope_fp8_quant.py:37-256 and its torch statement
// tests/test_fused_inv_rope_fp8_quant.py:150-198, which this kernel follows to the bit: the rotated
// tail is rounded to bf16 before it is quantised (the torch path does, the Triton kernel does not).
//
// One warp per (token, head) row in the A/B layout: the four quantisation groups are lanes 0-15 and
// 16-31 of each register; the rotary tail is register B of lanes 24-31.  HBM-bound: 1 KiB read,
// 512 + 16 bytes written per row.
#include "dsv4_common.cuh"

namespace dsv4 {
namespace {

struct InvRopeParams {
    const uint8_t* o;          // bf16 [N, H, 512], element strides below
    int64_t o_stride_token, o_stride_head;
    const int64_t* positions;  // [N]
    const float* cos_sin;      // fp32 rows of 64, row stride below
    int64_t cos_sin_stride;
    uint8_t* fp8;              // [G, N, hpg*512] e4m3
    uint8_t* scale;            // fp32 or int32, element (g, t, k) at g*scale_stride_group + t + k*padded_tokens
    int64_t scale_stride_group;
    int64_t num_tokens, padded_tokens;
    int32_t num_heads, heads_per_group;
    float eps;
    uint32_t heads_mul, heads_shift;  // fast division of a row index by num_heads (rows < 2^31)
    uint32_t hpg_mul, hpg_shift;      // fast division of a head index by heads_per_group
};

// Power-of-two scale >= s as (exponent byte, value): ceil(log2(max(s, 1e-10))) from the bit pattern.
__device__ __forceinline__ uint32_t pow2_ceil_code(float s) {
    const uint32_t u = __float_as_uint(fmaxf(s, 1e-10f));
    return ((u >> 23) & 0xffu) + ((u & 0x7fffffu) ? 1u : 0u);
}

__device__ __forceinline__ uint2 quant8_by(const float (&x)[8], float scale) {
    float q[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) q[i] = __fdiv_rn(x[i], scale);  // the e4m3 conversion saturates at +-448
    return make_uint2(pack_e4m3x4(q[0], q[1], q[2], q[3]), pack_e4m3x4(q[4], q[5], q[6], q[7]));
}

// 8 values times the exact reciprocal of a power-of-two scale (same result as dividing by it).
__device__ __forceinline__ uint2 quant8_pow2(const float (&x)[8], uint32_t code) {
    const float inv = __uint_as_float((254u - code) << 23);
    float q[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) q[i] = __fmul_rn(x[i], inv);
    return make_uint2(pack_e4m3x4(q[0], q[1], q[2], q[3]), pack_e4m3x4(q[4], q[5], q[6], q[7]));
}

// PACKED: power-of-two scales, the 4 UE8M0 bytes of a head packed into one int32.
// Each warp owns RPW consecutive (token, head) rows: all their loads are issued before the first is used.
template <int WARPS, int RPW, bool PACKED>
__global__ void __launch_bounds__(WARPS * 32) inv_rope_fp8_quant_kernel(const InvRopeParams p) {
    const int lane = threadIdx.x & 31;
    const uint32_t total = static_cast<uint32_t>(p.padded_tokens) * static_cast<uint32_t>(p.num_heads);
    const uint32_t row0 = (blockIdx.x * WARPS + (threadIdx.x >> 5)) * RPW;
    uint4 a[RPW], b[RPW];
    uint32_t token[RPW];
    int head[RPW];
#pragma unroll
    for (int i = 0; i < RPW; ++i) {
        const uint32_t row = row0 + i;
        token[i] = fast_div(row, p.heads_mul, p.heads_shift);
        head[i] = static_cast<int>(row - token[i] * static_cast<uint32_t>(p.num_heads));
        a[i] = b[i] = make_uint4(0u, 0u, 0u, 0u);
        if (row < total && token[i] < p.num_tokens) {
            const uint8_t* in = p.o + (static_cast<int64_t>(token[i]) * p.o_stride_token + head[i] * p.o_stride_head) * 2;
            a[i] = ld_stream16(in + 16 * lane);
            b[i] = ld_stream16(in + 512 + 16 * lane);
        }
    }
#pragma unroll
    for (int i = 0; i < RPW; ++i) {
        if (row0 + i >= total) break;
        const int group = static_cast<int>(fast_div(static_cast<uint32_t>(head[i]), p.hpg_mul, p.hpg_shift));
        const int head_in_group = head[i] - group * p.heads_per_group;
        uint8_t* scale_row = p.scale + (group * p.scale_stride_group + token[i]) * 4;
        if (token[i] >= p.num_tokens) {
            // rows of the token padding (scale columns are padded to a multiple of 4 tokens): zero scales
            if (PACKED) {
                if (lane == 0) *reinterpret_cast<uint32_t*>(scale_row + head_in_group * p.padded_tokens * 4) = 0u;
            } else if (lane < 4) {
                *reinterpret_cast<float*>(scale_row + (head_in_group * 4 + lane) * p.padded_tokens * 4) = 0.0f;
            }
            continue;
        }
        float xa[8], xb[8];
        unpack8(a[i], xa);
        unpack8(b[i], xb);
        if (lane >= kFirstRopeLane) {
            const float* cs = p.cos_sin + p.positions[token[i]] * p.cos_sin_stride + 4 * (lane - kFirstRopeLane);
            const float4 c4 = ld_readonly_f4(cs), s4 = ld_readonly_f4(cs + 32);
            const float c[4] = {c4.x, c4.y, c4.z, c4.w}, s[4] = {s4.x, s4.y, s4.z, s4.w};
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float e = xb[2 * j], o = xb[2 * j + 1];
                // inverse rotation, products rounded separately, then rounded to bf16 as the torch path does
                const float e2 = __fadd_rn(__fmul_rn(e, c[j]), __fmul_rn(o, s[j]));
                const float o2 = __fsub_rn(__fmul_rn(o, c[j]), __fmul_rn(e, s[j]));
                const uint32_t packed = pack_bf16x2(e2, o2);
                xb[2 * j] = bf16_lo(packed), xb[2 * j + 1] = bf16_hi(packed);
            }
        }
        float ma = 0.0f, mb = 0.0f;
#pragma unroll
        for (int k = 0; k < 8; ++k) ma = fmaxf(ma, fabsf(xa[k])), mb = fmaxf(mb, fabsf(xb[k]));
#pragma unroll
        for (int m = 1; m <= 8; m <<= 1) {
            ma = fmaxf(ma, __shfl_xor_sync(0xffffffffu, ma, m));
            mb = fmaxf(mb, __shfl_xor_sync(0xffffffffu, mb, m));
        }
        const float sa = __fmul_rn(fmaxf(ma, p.eps), 1.0f / 448.0f), sb = __fmul_rn(fmaxf(mb, p.eps), 1.0f / 448.0f);
        uint8_t* out = p.fp8 + (static_cast<int64_t>(group) * p.num_tokens + token[i]) * (static_cast<int64_t>(p.heads_per_group) * kRowBytes / 2) +
                       static_cast<int64_t>(head_in_group) * (kRowBytes / 2);
        if (PACKED) {
            const uint32_t code_a = pow2_ceil_code(sa), code_b = pow2_ceil_code(sb);
            st_global8(out + 8 * lane, quant8_pow2(xa, code_a));
            st_global8(out + 256 + 8 * lane, quant8_pow2(xb, code_b));
            // chunk k of the head in byte k: groups 0,1 from register A (lanes 0 / 16), 2,3 from B
            const uint32_t word = (__shfl_sync(0xffffffffu, code_a, 0) & 0xffu) | ((__shfl_sync(0xffffffffu, code_a, 16) & 0xffu) << 8) |
                                  ((__shfl_sync(0xffffffffu, code_b, 0) & 0xffu) << 16) |
                                  ((__shfl_sync(0xffffffffu, code_b, 16) & 0xffu) << 24);
            if (lane == 0) *reinterpret_cast<uint32_t*>(scale_row + head_in_group * p.padded_tokens * 4) = word;
        } else {
            st_global8(out + 8 * lane, quant8_by(xa, sa));
            st_global8(out + 256 + 8 * lane, quant8_by(xb, sb));
            if ((lane & 15) == 0) {
                const int k = head_in_group * 4 + (lane >> 4);
                *reinterpret_cast<float*>(scale_row + k * p.padded_tokens * 4) = sa;
                *reinterpret_cast<float*>(scale_row + (k + 2) * p.padded_tokens * 4) = sb;
            }
        }
    }
}

}  // namespace

cudaError_t launch_inv_rope_fp8_quant(const void* o, int64_t o_stride_token, int64_t o_stride_head, const int64_t* positions,
                                      const float* cos_sin, int64_t cos_sin_stride, void* fp8, void* scale,
                                      int64_t scale_stride_group, int64_t num_tokens, int64_t padded_tokens, int num_heads,
                                      int heads_per_group, float eps, int packed, cudaStream_t stream) {
    constexpr int WARPS = 4, RPW = 2;
    const int64_t rows = padded_tokens * num_heads;
    if (rows == 0) return cudaSuccess;
    const int64_t grid = (rows + WARPS * RPW - 1) / (WARPS * RPW);
    if (grid > 0x7fffffffLL) return cudaErrorInvalidConfiguration;
    InvRopeParams p{};
    p.o = static_cast<const uint8_t*>(o), p.o_stride_token = o_stride_token, p.o_stride_head = o_stride_head;
    p.positions = positions, p.cos_sin = cos_sin, p.cos_sin_stride = cos_sin_stride;
    p.fp8 = static_cast<uint8_t*>(fp8), p.scale = static_cast<uint8_t*>(scale), p.scale_stride_group = scale_stride_group;
    p.num_tokens = num_tokens, p.padded_tokens = padded_tokens, p.num_heads = num_heads, p.heads_per_group = heads_per_group;
    p.eps = eps;
    if (rows >= (1LL << 31)) return cudaErrorInvalidConfiguration;
    make_fast_divisor(static_cast<uint32_t>(num_heads), &p.heads_mul, &p.heads_shift);
    make_fast_divisor(static_cast<uint32_t>(heads_per_group), &p.hpg_mul, &p.hpg_shift);
    if (packed) inv_rope_fp8_quant_kernel<WARPS, RPW, true><<<static_cast<unsigned>(grid), WARPS * 32, 0, stream>>>(p);
    else inv_rope_fp8_quant_kernel<WARPS, RPW, false><<<static_cast<unsigned>(grid), WARPS * 32, 0, stream>>>(p);
    count_launch();
    return cudaGetLastError();
}

}  // namespace dsv4
