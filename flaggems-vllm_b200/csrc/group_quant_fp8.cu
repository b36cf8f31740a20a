// per_token_group_quant_fp8: FP8 e4m3 quantisation of activations x [M, K] (bf16) in groups of group_size
// consecutive values with one fp32 scale per group - the quantiser in front of the FP8 projections of the attention
// layer (the epilogue quantiser is this operator with the inverse rotation in front of it).
// Reference: src/flaggems_vllm/ops/per_token_group_quant_fp8.py:25-330 and its torch statement
// tests/test_per_token_group_quant_fp8.py:53-89:
//   scale = max(amax, eps) * (1/448), rounded up to a power of two when scale_ue8m0; x_q = e4m3(clamp(x / scale)).
//   The statement clamps the maximum while it still has the input's type, so eps takes effect rounded to bf16.
// Also `act_quant_triton` (src/flaggems_vllm/ops/act_quant.py:22-175, statement tests/test_act_quant.py:49-99): the same
// operator with the maximum clamped at 1e-4 in fp32 and x * (1/scale) in place of the division.
// HBM traffic: 2 bytes read, 1 byte + 4/group_size bytes written per value.
#include <cstring>

#include "dsv4_common.cuh"

namespace dsv4 {
namespace {

struct GroupQuantParams {
    const uint8_t* x;  // bf16 [M, K], row stride in elements
    int64_t x_stride;
    uint8_t* out;  // e4m3 [M, K], contiguous
    float* scales;  // element (row, group) at row*scale_stride_row + group*scale_stride_group
    int64_t scale_stride_row, scale_stride_group;
    int64_t num_groups;  // M * K / group_size
    int32_t groups_per_row, group_size;
    float eps;
    uint32_t gpr_mul, gpr_shift;  // fast division of a group index by groups_per_row
};

// LANES adjacent lanes per group, CHUNKS x 8 values per lane (group_size = LANES * CHUNKS * 8), U groups per lane
// group in flight.  UE8M0: power-of-two scales (exact reciprocal multiply); DIVISION: how x / scale is formed otherwise
// (IEEE division, the verified reciprocal-and-correct division for the default eps, or x * (1/scale) for `act_quant`).
template <int WARPS, int LANES, int CHUNKS, int U, bool UE8M0, int DIVISION>
__global__ void __launch_bounds__(WARPS * 32) group_quant_fp8_kernel(const GroupQuantParams p) {
    constexpr int kGroups = 32 / LANES;
    const int lane = threadIdx.x & 31;
    const int sub = lane % LANES;
    const int64_t first = (static_cast<int64_t>(blockIdx.x) * WARPS + (threadIdx.x >> 5)) * (kGroups * U) + lane / LANES;
    uint4 v[U][CHUNKS];
    int64_t row[U];
    int32_t col[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
        const int64_t g = first + u * kGroups;
        row[u] = 0, col[u] = 0;
#pragma unroll
        for (int c = 0; c < CHUNKS; ++c) v[u][c] = make_uint4(0u, 0u, 0u, 0u);
        if (g < p.num_groups) {
            row[u] = fast_div(static_cast<uint32_t>(g), p.gpr_mul, p.gpr_shift);
            col[u] = static_cast<int32_t>(g - row[u] * p.groups_per_row);
            const uint8_t* src = p.x + (row[u] * p.x_stride + static_cast<int64_t>(col[u]) * p.group_size) * 2;
#pragma unroll
            for (int c = 0; c < CHUNKS; ++c) v[u][c] = ld_stream16(src + 16 * (sub + c * LANES));
        }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
        const int64_t g = first + u * kGroups;
        // |.| maximum on the packed words (even and odd elements side by side), then across the group's lanes
        uint32_t pk = max_abs_bf16x2(max_abs_bf16x2(v[u][0].x, v[u][0].y), max_abs_bf16x2(v[u][0].z, v[u][0].w));
#pragma unroll
        for (int c = 1; c < CHUNKS; ++c)
            pk = max_abs_bf16x2(pk, max_abs_bf16x2(max_abs_bf16x2(v[u][c].x, v[u][c].y), max_abs_bf16x2(v[u][c].z, v[u][c].w)));
        pk &= 0x7fff7fffu;
#pragma unroll
        for (int m = 1; m < LANES; m <<= 1) pk = max_bf16x2(pk, __shfl_xor_sync(0xffffffffu, pk, m));
        const float amax = fmaxf(bf16_lo(pk), bf16_hi(pk));
        float scale = __fmul_rn(fmaxf(amax, p.eps), 1.0f / 448.0f);
        uint32_t code = 0u;
        if (UE8M0) {
            code = pow2_ceil_code(scale);
            scale = __uint_as_float(code << 23);
        }
        const bool two_term = !UE8M0 && DIVISION == kDivideFast && __all_sync(0xffffffffu, scale <= kTwoTermMaxScale);
        if (g >= p.num_groups) continue;
        uint8_t* dst = p.out + g * p.group_size;
        if (UE8M0) {
#pragma unroll
            for (int c = 0; c < CHUNKS; ++c) st_global8(dst + 8 * (sub + c * LANES), quant8_pow2(v[u][c], code));
        } else {
            // one warp-uniform choice of the division form per pass (see ScaleDivider); lanes past the last group
            // have left the loop body above only after the vote, so every lane takes part in it
            const ScaleDivider<DIVISION> by_scale(scale);
            if (two_term) {
#pragma unroll
                for (int c = 0; c < CHUNKS; ++c) st_global8(dst + 8 * (sub + c * LANES), quant8_by<DIVISION, true>(v[u][c], by_scale));
            } else {
#pragma unroll
                for (int c = 0; c < CHUNKS; ++c) st_global8(dst + 8 * (sub + c * LANES), quant8_by<DIVISION, false>(v[u][c], by_scale));
            }
        }
        if (sub == 0) p.scales[row[u] * p.scale_stride_row + col[u] * p.scale_stride_group] = scale;
    }
}

// Any group size and alignment: one warp per group, element by element.
template <int WARPS>
__global__ void __launch_bounds__(WARPS * 32) group_quant_fp8_scalar_kernel(const GroupQuantParams p, const int ue8m0, const int reciprocal) {
    const int lane = threadIdx.x & 31;
    const int64_t g = static_cast<int64_t>(blockIdx.x) * WARPS + (threadIdx.x >> 5);
    if (g >= p.num_groups) return;
    const int64_t row = g / p.groups_per_row;
    const int64_t col = g - row * p.groups_per_row;
    const uint16_t* src = reinterpret_cast<const uint16_t*>(p.x) + row * p.x_stride + col * p.group_size;
    float amax = 0.0f;
    for (int i = lane; i < p.group_size; i += 32) amax = fmaxf(amax, fabsf(bf16_lo(src[i])));
#pragma unroll
    for (int m = 16; m > 0; m >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, m));
    float scale = __fmul_rn(fmaxf(amax, p.eps), 1.0f / 448.0f);
    if (ue8m0) scale = __uint_as_float(pow2_ceil_code(scale) << 23);
    uint8_t* dst = p.out + g * p.group_size;
    const float recip = __frcp_rn(scale);
    for (int i = lane; i < p.group_size; i += 32)
        dst[i] = static_cast<uint8_t>(pack_e4m3x4(reciprocal ? __fmul_rn(bf16_lo(src[i]), recip) : __fdiv_rn(bf16_lo(src[i]), scale), 0.0f, 0.0f, 0.0f) & 0xffu);
    if (lane == 0) p.scales[row * p.scale_stride_row + col * p.scale_stride_group] = scale;
}

template <int LANES, int CHUNKS>
void launch_vector(const GroupQuantParams& p, bool ue8m0, int division, cudaStream_t stream) {
    constexpr int WARPS = 4, U = CHUNKS == 1 ? 4 : 2;
    const int64_t per_cta = static_cast<int64_t>(WARPS) * (32 / LANES) * U;
    const unsigned grid = static_cast<unsigned>((p.num_groups + per_cta - 1) / per_cta);
    if (ue8m0) group_quant_fp8_kernel<WARPS, LANES, CHUNKS, U, true, kDivideIeee><<<grid, WARPS * 32, 0, stream>>>(p);
    else if (division == kDivideFast) group_quant_fp8_kernel<WARPS, LANES, CHUNKS, U, false, kDivideFast><<<grid, WARPS * 32, 0, stream>>>(p);
    else if (division == kMultiplyReciprocal) group_quant_fp8_kernel<WARPS, LANES, CHUNKS, U, false, kMultiplyReciprocal><<<grid, WARPS * 32, 0, stream>>>(p);
    else group_quant_fp8_kernel<WARPS, LANES, CHUNKS, U, false, kDivideIeee><<<grid, WARPS * 32, 0, stream>>>(p);
}

}  // namespace

cudaError_t launch_group_quant_fp8(const void* x, int64_t x_stride, void* out, float* scales, int64_t scale_stride_row,
                                   int64_t scale_stride_group, int64_t num_rows, int64_t num_cols, int group_size, float eps, int ue8m0,
                                   int act_quant_rules, cudaStream_t stream) {
    const int64_t groups_per_row = num_cols / group_size;
    const int64_t num_groups = num_rows * groups_per_row;
    if (num_groups == 0) return cudaSuccess;
    if (num_groups >= (1LL << 31)) return cudaErrorInvalidConfiguration;
    GroupQuantParams p{};
    p.x = static_cast<const uint8_t*>(x), p.x_stride = x_stride, p.out = static_cast<uint8_t*>(out), p.scales = scales;
    p.scale_stride_row = scale_stride_row, p.scale_stride_group = scale_stride_group, p.num_groups = num_groups;
    p.groups_per_row = static_cast<int32_t>(groups_per_row), p.group_size = group_size;
    p.eps = eps;
    if (!act_quant_rules) {  // eps rounded to bf16 (nearest even), as a clamp of a bf16 tensor applies it
        uint32_t bits;
        memcpy(&bits, &eps, 4);
        bits = (bits + 0x7fffu + ((bits >> 16) & 1u)) & 0xffff0000u;
        memcpy(&p.eps, &bits, 4);
    }
    make_fast_divisor(static_cast<uint32_t>(groups_per_row), &p.gpr_mul, &p.gpr_shift);
    const auto addr = [](const void* q) { return reinterpret_cast<uintptr_t>(q); };
    const bool vec = addr(x) % 16 == 0 && x_stride % 8 == 0 && addr(out) % 8 == 0 &&
                     (group_size == 64 || group_size == 128 || group_size == 256 || group_size == 512);
    const int division = act_quant_rules ? kMultiplyReciprocal : (eps == 1e-10f ? kDivideFast : kDivideIeee);
    if (!vec) {
        constexpr int WARPS = 4;
        group_quant_fp8_scalar_kernel<WARPS><<<static_cast<unsigned>((num_groups + WARPS - 1) / WARPS), WARPS * 32, 0, stream>>>(p, ue8m0, act_quant_rules);
    } else if (group_size == 64) {
        launch_vector<8, 1>(p, ue8m0 != 0, division, stream);
    } else if (group_size == 128) {
        launch_vector<16, 1>(p, ue8m0 != 0, division, stream);
    } else if (group_size == 256) {
        launch_vector<32, 1>(p, ue8m0 != 0, division, stream);
    } else {
        launch_vector<32, 2>(p, ue8m0 != 0, division, stream);
    }
    count_launch();
    return cudaGetLastError();
}

}  // namespace dsv4
