// fused_inv_rope_fp8_quant: the attention epilogue that mirrors the prologue - inverse GPT-J RoPE on
// the rotary tail of the attention output o [N, H, 512], then FP8 e4m3 quantisation in groups of 128
// with one scale per group (fp32 = amax/448, or a power of two packed as UE8M0 bytes).
// Reference: src/flaggems_vllm/ops/fused_inv_rope_fp8_quant.py:37-256 and its torch statement
// tests/test_fused_inv_rope_fp8_quant.py:150-198, which this kernel follows to the bit: the rotated
// tail is rounded to bf16 before it is quantised (the torch path does, the Triton kernel does not).
//
// HBM traffic: 1 KiB read, 512 + 16 bytes written per (token, head) row.
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

// PACKED: power-of-two scales, the 4 UE8M0 bytes of a head packed into one int32.
// A warp owns kHeadsPerTask consecutive heads of one token and walks them U at a time.  Rows are held in the
// A/B/T layout (A: 16 B per lane, B: 16 B in lanes 0-23, T: the 4-byte rotary pair 448+2l, 449+2l of lane l), so
// every lane rotates exactly one pair with a cosine and sine it loaded once for the whole task.  The four
// quantisation groups of 128 are: A lanes 0-15, A lanes 16-31, B lanes 0-15, and B lanes 16-23 together with T.
constexpr int kHeadsPerTask = 16;
#ifndef DSV4_INVROPE_UE8M0_CTAS
#define DSV4_INVROPE_UE8M0_CTAS 7  // CTAs per SM of the UE8M0-scale instantiation (72 registers with two passes in flight)
#endif
#ifndef DSV4_INVROPE_FP32_CTAS
#define DSV4_INVROPE_FP32_CTAS 8  // CTAs per SM of the fp32-scale instantiation (64 registers with two passes in flight)
#endif

// FASTDIV (fp32-scale mode only): see ScaleDivider.
// PREFETCH: two passes of U heads in flight - the loads of the next pass go out before the current one is worked on, so
// a warp always has rows on their way while it computes (UE8M0 scales: 267 -> 256 us on 1 Mi rows; fp32 scales, once the
// per-head address arithmetic was reduced to increments: 272 -> 269 us).
template <int WARPS, bool PACKED, bool FASTDIV, int U, int MIN_CTAS, bool PREFETCH>
__global__ void __launch_bounds__(WARPS * 32, MIN_CTAS) inv_rope_fp8_quant_kernel(const InvRopeParams p, const uint32_t tasks_per_token,
                                                                      const uint32_t tpt_mul, const uint32_t tpt_shift) {
    const int lane = threadIdx.x & 31;
    const uint32_t task = blockIdx.x * WARPS + (threadIdx.x >> 5);
    if (task >= static_cast<uint32_t>(p.padded_tokens) * tasks_per_token) return;
    const uint32_t token = fast_div(task, tpt_mul, tpt_shift);
    const int head_begin = static_cast<int>(task - token * tasks_per_token) * kHeadsPerTask;
    const int head_end = head_begin + kHeadsPerTask < p.num_heads ? head_begin + kHeadsPerTask : p.num_heads;
    if (token >= p.num_tokens) {
        // token padding of the scale storage (a multiple of 4 tokens): zero scales
        for (int head = head_begin; head < head_end; ++head) {
            const int group = static_cast<int>(fast_div(static_cast<uint32_t>(head), p.hpg_mul, p.hpg_shift));
            const int head_in_group = head - group * p.heads_per_group;
            uint8_t* scale_row = p.scale + (group * p.scale_stride_group + token) * 4;
            if (PACKED) {
                if (lane == 0) *reinterpret_cast<uint32_t*>(scale_row + head_in_group * p.padded_tokens * 4) = 0u;
            } else if (lane < 4) {
                *reinterpret_cast<float*>(scale_row + (head_in_group * 4 + lane) * p.padded_tokens * 4) = 0.0f;
            }
        }
        return;
    }
    const float* cs = p.cos_sin + p.positions[token] * p.cos_sin_stride;
    const float c = cs[lane], sn = cs[32 + lane];
    const uint8_t* in_token = p.o + static_cast<int64_t>(token) * p.o_stride_token * 2;
    uint4 a[U], b[U], a_next[U], b_next[U];
    uint32_t tail[U], tail_next[U];
    const auto load_pass = [&](int h0, uint4 (&ra)[U], uint4 (&rb)[U], uint32_t (&rt)[U]) {
#pragma unroll
        for (int u = 0; u < U; ++u) {
            ra[u] = rb[u] = make_uint4(0u, 0u, 0u, 0u);
            rt[u] = 0u;
            if (h0 + u < head_end) {
                const uint8_t* in = in_token + (h0 + u) * p.o_stride_head * 2;
                ra[u] = ld_stream16(in + 16 * lane);
                if (lane < kFirstRopeLane) rb[u] = ld_stream16(in + 512 + 16 * lane);
                rt[u] = ld_stream4(in + 2 * kNopeDim + 4 * lane);
            }
        }
    };
    // Output addresses advance by constants from one head to the next and are recomputed only where a new group of heads
    // begins: `out` = the head's 512 e4m3 bytes, `scale_at` = its first scale (this lane's half of the four in fp32 mode).
    int group = static_cast<int>(fast_div(static_cast<uint32_t>(head_begin), p.hpg_mul, p.hpg_shift));
    int head_in_group = head_begin - group * p.heads_per_group;
    const int64_t group_bytes = static_cast<int64_t>(p.heads_per_group) * (kRowBytes / 2);
    const int64_t scale_column = p.padded_tokens * 4;                       // bytes between scale columns of one token
    const int64_t scale_step = PACKED ? scale_column : 4 * scale_column;    // ... between consecutive heads
    const int64_t lane_scale = PACKED ? 0 : (lane >> 4) * scale_column;     // fp32: lanes 0 / 16 store groups 0,2 / 1,3
    const auto group_out = [&](int g) { return p.fp8 + (static_cast<int64_t>(g) * p.num_tokens + token) * group_bytes; };
    const auto group_scale = [&](int g) { return p.scale + (g * p.scale_stride_group + token) * 4 + lane_scale; };
    uint8_t* out = group_out(group) + static_cast<int64_t>(head_in_group) * (kRowBytes / 2);
    uint8_t* scale_at = group_scale(group) + head_in_group * scale_step;
    load_pass(head_begin, a, b, tail);
    for (int h0 = head_begin; h0 < head_end; h0 += U) {
        if (PREFETCH) load_pass(h0 + U, a_next, b_next, tail_next);  // past the last head of the task: nothing is loaded
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int head = h0 + u;
            if (head >= head_end) break;
            // inverse rotation of the lane's pair, products rounded separately, then to bf16 as the torch path does
            const float e = bf16_lo(tail[u]), o = bf16_hi(tail[u]);
            const uint32_t rot = pack_bf16x2(__fadd_rn(__fmul_rn(e, c), __fmul_rn(o, sn)), __fsub_rn(__fmul_rn(o, c), __fmul_rn(e, sn)));
            const float te = bf16_lo(rot), to = bf16_hi(rot);
            // Group maxima on the packed words: |.| maxima of the even and the odd elements side by side (the sign
            // bits of the intermediate words are meaningless and cleared at the end).
            const uint32_t pa = max_abs_bf16x2(max_abs_bf16x2(a[u].x, a[u].y), max_abs_bf16x2(a[u].z, a[u].w));
            uint32_t pb = max_abs_bf16x2(max_abs_bf16x2(b[u].x, b[u].y), max_abs_bf16x2(b[u].z, b[u].w));
            // Group 3 = B of lanes 16-23 and all of T: the upper half-warp folds its own pair and the pair of the
            // lane 16 below into its B maximum, so that one packed reduction over 16 lanes serves all four groups.
            const uint32_t rot_other = __shfl_xor_sync(0xffffffffu, rot, 16);
            if (lane >= 16) pb = max_abs_bf16x2(max_abs_bf16x2(pb, rot), rot_other);
            // (A even | B even) against (A odd | B odd): the A maximum in the low half, the B maximum in the high half
            uint32_t both = max_abs_bf16x2(__byte_perm(pa, pb, 0x5410), __byte_perm(pa, pb, 0x7632)) & 0x7fff7fffu;
#pragma unroll
            for (int m = 1; m <= 8; m <<= 1) both = max_bf16x2(both, __shfl_xor_sync(0xffffffffu, both, m));
            const uint32_t both_other = __shfl_xor_sync(0xffffffffu, both, 16);
            const float ma = bf16_lo(both), mb = bf16_hi(both);
            const float m3 = lane >= 16 ? mb : bf16_hi(both_other);
            const float sa = __fmul_rn(fmaxf(ma, p.eps), 1.0f / 448.0f), sb = __fmul_rn(fmaxf(mb, p.eps), 1.0f / 448.0f);
            const float s3 = __fmul_rn(fmaxf(m3, p.eps), 1.0f / 448.0f);
            if (PACKED) {
                const uint32_t code_a = pow2_ceil_code(sa), code_b = pow2_ceil_code(sb), code_3 = pow2_ceil_code(s3);
                st_global8(out + 8 * lane, quant8_pow2(a[u], code_a));
                if (lane < kFirstRopeLane) st_global8(out + 256 + 8 * lane, quant8_pow2(b[u], code_b));
                const float inv3 = __uint_as_float((254u - code_3) << 23);
                *reinterpret_cast<uint16_t*>(out + kNopeDim + 2 * lane) =
                    static_cast<uint16_t>(pack_e4m3x4(__fmul_rn(te, inv3), __fmul_rn(to, inv3), 0.f, 0.f));
                // chunk k of the head in byte k: lane 0 holds the codes of groups 0 and 2, lane 16 those of 1 and 3
                const uint32_t mine = code_a | (code_b << 16);
                const uint32_t word = mine | (__shfl_xor_sync(0xffffffffu, mine, 16) << 8);
                if (lane == 0) *reinterpret_cast<uint32_t*>(scale_at) = word;
            } else {
                // the three-instruction form of the fast division for every scale: measured here, a warp-uniform choice
                // between it and the two-instruction form was no faster (296 us against 294 us on 1 Mi rows)
                constexpr int kDivision = FASTDIV ? kDivideFast : kDivideIeee;
                const ScaleDivider<kDivision> by_a(sa), by_b(sb), by_3(s3);
                st_global8(out + 8 * lane, quant8_by<kDivision, false>(a[u], by_a));
                if (lane < kFirstRopeLane) st_global8(out + 256 + 8 * lane, quant8_by<kDivision, false>(b[u], by_b));
                *reinterpret_cast<uint16_t*>(out + kNopeDim + 2 * lane) = static_cast<uint16_t>(
                    pack_e4m3x4(by_3.template quotient<false>(te), by_3.template quotient<false>(to), 0.f, 0.f));
                if ((lane & 15) == 0) {
                    *reinterpret_cast<float*>(scale_at) = sa;
                    *reinterpret_cast<float*>(scale_at + 2 * scale_column) = sb;  // lane 16: sb is s3
                }
            }
            // on to the next head
            out += kRowBytes / 2, scale_at += scale_step;
            if (++head_in_group == p.heads_per_group) {
                head_in_group = 0, ++group;
                out = group_out(group), scale_at = group_scale(group);
            }
        }
        if (PREFETCH) {
#pragma unroll
            for (int u = 0; u < U; ++u) a[u] = a_next[u], b[u] = b_next[u], tail[u] = tail_next[u];
        } else {
            load_pass(h0 + U, a, b, tail);
        }
    }
}

// Any geometry the reference wrapper accepts (head_dim = nope + rope a multiple of the group size, the rotary tail
// ending the last group, even group size): one warp per (token, head), one group after the other, two passes over a
// group (maximum, then quantise; the rotation is recomputed, which is deterministic).  Same arithmetic as above: rotated
// values rounded to bf16 before quantising, fp32 scales divide (IEEE), power-of-two scales multiply by the exact
// reciprocal.  Packed scales need four groups per head: one int32 per head is the only layout in which the reference's
// kernel and its allocation agree (src/flaggems_vllm/ops/fused_inv_rope_fp8_quant.py:133-143, 206-217).
struct InvRopeGeometry {
    int32_t nope_dim, rope_dim, group, chunks;
};

template <int WARPS, bool PACKED>
__global__ void __launch_bounds__(WARPS * 32) inv_rope_fp8_quant_any_kernel(const InvRopeParams p, const InvRopeGeometry geo) {
    const int lane = threadIdx.x & 31;
    const int64_t row = static_cast<int64_t>(blockIdx.x) * WARPS + (threadIdx.x >> 5);
    if (row >= p.padded_tokens * p.num_heads) return;
    const int64_t token = row / p.num_heads;
    const int head = static_cast<int>(row - token * p.num_heads);
    const int group = head / p.heads_per_group, head_in_group = head - group * p.heads_per_group;
    uint8_t* scale_row = p.scale + (group * p.scale_stride_group + token) * 4;
    if (token >= p.num_tokens) {  // token padding of the scale storage: zero scales
        if (PACKED) {
            if (lane == 0) *reinterpret_cast<uint32_t*>(scale_row + static_cast<int64_t>(head_in_group) * p.padded_tokens * 4) = 0u;
        } else if (lane < geo.chunks) {
            *reinterpret_cast<float*>(scale_row + (static_cast<int64_t>(head_in_group) * geo.chunks + lane) * p.padded_tokens * 4) = 0.0f;
        }
        return;
    }
    const int head_dim = geo.nope_dim + geo.rope_dim, half_rope = geo.rope_dim / 2;
    const float* cs = p.cos_sin + p.positions[token] * p.cos_sin_stride;
    const uint16_t* in = reinterpret_cast<const uint16_t*>(p.o) + token * p.o_stride_token + static_cast<int64_t>(head) * p.o_stride_head;
    uint8_t* out = p.fp8 + (static_cast<int64_t>(group) * p.num_tokens + token) * (static_cast<int64_t>(p.heads_per_group) * head_dim) +
                   static_cast<int64_t>(head_in_group) * head_dim;
    // the pair (2j, 2j+1) of the head after the inverse rotation (if it lies in the rotary tail) and the bf16 rounding
    const auto pair_at = [&](int e0, float* a, float* b) {
        const float e = bf16_lo(in[e0]), o = bf16_lo(in[e0 + 1]);
        if (e0 >= geo.nope_dim) {
            const int j = (e0 - geo.nope_dim) >> 1;
            const float c = cs[j], sn = cs[half_rope + j];
            const uint32_t rot = pack_bf16x2(__fadd_rn(__fmul_rn(e, c), __fmul_rn(o, sn)), __fsub_rn(__fmul_rn(o, c), __fmul_rn(e, sn)));
            *a = bf16_lo(rot), *b = bf16_hi(rot);
        } else {
            *a = e, *b = o;
        }
    };
    uint32_t word = 0;
    for (int k = 0; k < geo.chunks; ++k) {
        float amax = 0.0f;
        for (int pr = lane; pr < geo.group / 2; pr += 32) {
            float a, b;
            pair_at(k * geo.group + 2 * pr, &a, &b);
            amax = fmaxf(amax, fmaxf(fabsf(a), fabsf(b)));
        }
#pragma unroll
        for (int m = 16; m > 0; m >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, m));
        float scale = __fmul_rn(fmaxf(amax, p.eps), 1.0f / 448.0f);
        float inv = 0.0f;
        if (PACKED) {
            const uint32_t code = pow2_ceil_code(scale);
            word |= code << (8 * k);
            inv = __uint_as_float((254u - code) << 23);
        }
        for (int pr = lane; pr < geo.group / 2; pr += 32) {
            const int e0 = k * geo.group + 2 * pr;
            float a, b;
            pair_at(e0, &a, &b);
            const float qa = PACKED ? __fmul_rn(a, inv) : __fdiv_rn(a, scale), qb = PACKED ? __fmul_rn(b, inv) : __fdiv_rn(b, scale);
            *reinterpret_cast<uint16_t*>(out + e0) = static_cast<uint16_t>(pack_e4m3x4(qa, qb, 0.f, 0.f));
        }
        if (!PACKED && lane == 0)
            *reinterpret_cast<float*>(scale_row + (static_cast<int64_t>(head_in_group) * geo.chunks + k) * p.padded_tokens * 4) = scale;
    }
    if (PACKED && lane == 0) *reinterpret_cast<uint32_t*>(scale_row + static_cast<int64_t>(head_in_group) * p.padded_tokens * 4) = word;
}

}  // namespace

cudaError_t launch_inv_rope_fp8_quant_any(const void* o, int64_t o_stride_token, int64_t o_stride_head, const int64_t* positions,
                                          const float* cos_sin, int64_t cos_sin_stride, void* fp8, void* scale,
                                          int64_t scale_stride_group, int64_t num_tokens, int64_t padded_tokens, int num_heads,
                                          int heads_per_group, int nope_dim, int rope_dim, int group_size, float eps, int packed,
                                          cudaStream_t stream) {
    constexpr int WARPS = 4;
    const int64_t rows = padded_tokens * num_heads;
    if (rows == 0) return cudaSuccess;
    const int64_t grid = (rows + WARPS - 1) / WARPS;
    if (grid > 0x7fffffffLL) return cudaErrorInvalidConfiguration;
    InvRopeParams p{};
    p.o = static_cast<const uint8_t*>(o), p.o_stride_token = o_stride_token, p.o_stride_head = o_stride_head;
    p.positions = positions, p.cos_sin = cos_sin, p.cos_sin_stride = cos_sin_stride;
    p.fp8 = static_cast<uint8_t*>(fp8), p.scale = static_cast<uint8_t*>(scale), p.scale_stride_group = scale_stride_group;
    p.num_tokens = num_tokens, p.padded_tokens = padded_tokens, p.num_heads = num_heads, p.heads_per_group = heads_per_group;
    p.eps = eps;
    const InvRopeGeometry geo{nope_dim, rope_dim, group_size, (nope_dim + rope_dim) / group_size};
    if (packed) inv_rope_fp8_quant_any_kernel<WARPS, true><<<static_cast<unsigned>(grid), WARPS * 32, 0, stream>>>(p, geo);
    else inv_rope_fp8_quant_any_kernel<WARPS, false><<<static_cast<unsigned>(grid), WARPS * 32, 0, stream>>>(p, geo);
    count_launch();
    return cudaGetLastError();
}

cudaError_t launch_inv_rope_fp8_quant(const void* o, int64_t o_stride_token, int64_t o_stride_head, const int64_t* positions,
                                      const float* cos_sin, int64_t cos_sin_stride, void* fp8, void* scale,
                                      int64_t scale_stride_group, int64_t num_tokens, int64_t padded_tokens, int num_heads,
                                      int heads_per_group, float eps, int packed, cudaStream_t stream) {
    constexpr int WARPS = 4;
    const int64_t rows = padded_tokens * num_heads;
    if (rows == 0) return cudaSuccess;
    const int64_t tasks_per_token = (num_heads + kHeadsPerTask - 1) / kHeadsPerTask;
    const int64_t tasks = padded_tokens * tasks_per_token;
    const int64_t grid = (tasks + WARPS - 1) / WARPS;
    if (grid > 0x7fffffffLL || tasks >= (1LL << 31)) return cudaErrorInvalidConfiguration;
    InvRopeParams p{};
    p.o = static_cast<const uint8_t*>(o), p.o_stride_token = o_stride_token, p.o_stride_head = o_stride_head;
    p.positions = positions, p.cos_sin = cos_sin, p.cos_sin_stride = cos_sin_stride;
    p.fp8 = static_cast<uint8_t*>(fp8), p.scale = static_cast<uint8_t*>(scale), p.scale_stride_group = scale_stride_group;
    p.num_tokens = num_tokens, p.padded_tokens = padded_tokens, p.num_heads = num_heads, p.heads_per_group = heads_per_group;
    p.eps = eps;
    make_fast_divisor(static_cast<uint32_t>(num_heads), &p.heads_mul, &p.heads_shift);
    make_fast_divisor(static_cast<uint32_t>(heads_per_group), &p.hpg_mul, &p.hpg_shift);
    uint32_t tpt_mul, tpt_shift;
    make_fast_divisor(static_cast<uint32_t>(tasks_per_token), &tpt_mul, &tpt_shift);
    const unsigned g = static_cast<unsigned>(grid);
    const uint32_t tpt = static_cast<uint32_t>(tasks_per_token);
    // Heads in flight per warp and CTAs per SM, measured on 1 Mi rows.  UE8M0 mode, two passes of 2 heads in flight: 7 CTAs
    // (72 registers) 256 us, 8 CTAs (64 registers, 8 bytes spilled) 257 us, 6 CTAs 262 us; one pass in flight at 10 CTAs
    // 265-282 us.  fp32-scale mode: two passes at 8 CTAs (64 registers) 269 us, at 7 CTAs 270 us; one pass at 10 CTAs
    // (48 registers) 272 us, at 9 CTAs 274 us, at 11 CTAs 301 us.
    if (packed) inv_rope_fp8_quant_kernel<WARPS, true, false, 2, DSV4_INVROPE_UE8M0_CTAS, true><<<g, WARPS * 32, 0, stream>>>(p, tpt, tpt_mul, tpt_shift);
    else if (eps == 1e-10f) inv_rope_fp8_quant_kernel<WARPS, false, true, 2, DSV4_INVROPE_FP32_CTAS, true><<<g, WARPS * 32, 0, stream>>>(p, tpt, tpt_mul, tpt_shift);
    else inv_rope_fp8_quant_kernel<WARPS, false, false, 2, 8, false><<<g, WARPS * 32, 0, stream>>>(p, tpt, tpt_mul, tpt_shift);
    count_launch();
    return cudaGetLastError();
}

}  // namespace dsv4
