// fused_indexer_q_rope_quant: the sparse-indexer prologue that runs beside the attention prologue -
// GPT-J RoPE on the last rot_dim values of every index-q head (rounded to bf16), then either
//   FP8:   one power-of-two scale per (token, head), e4m3 values, scale folded into the head weight, or
//   MXFP4: one UE8M0 scale per 32 values, e2m1 values packed two per byte (cvt.rn.satfinite.e2m1x2.f32,
//          an sm_100 instruction), weights scaled by softmax_scale*head_scale only.
// Reference: src/flaggems_vllm/ops/fused_indexer_q_rope_quant.py:69-410 and its torch statement
// tests/test_fused_indexer_q_rope_quant.py:48-113.
// Fast shape: head_dim/8 lanes per (token, head) row, 16 bytes per lane, several rows per warp instruction.
// General shape: one warp per row; lane l keeps E = head_dim/32 consecutive values (E/2 rotary pairs).
#include "dsv4_common.cuh"

namespace dsv4 {
namespace {

struct IndexerQParams {
    const int64_t* positions;
    const uint8_t* q;  // bf16 [T, H, D], element strides
    int64_t q_stride0, q_stride1;
    const uint8_t* cos_sin;  // [max_pos, rot_dim] fp32 or bf16, row stride in elements
    int64_t cos_sin_stride;
    int32_t cos_sin_bf16, rot_dim;
    uint8_t* out;  // fp8: [T, H, D] bytes; fp4: [T, H, D/2] bytes (strides in bytes)
    int64_t out_stride0, out_stride1;
    uint8_t* scales;  // fp4 only: [T, H, D/32] bytes
    int64_t scale_stride0, scale_stride1;
    const uint8_t* weights;  // [T, H], row stride in elements; dtype code 0 bf16, 1 fp16, 2 fp32
    int64_t weights_stride;
    int32_t weights_dtype;
    float* weights_out;  // fp32 [T, H], row stride in elements
    int64_t weights_out_stride;
    float softmax_scale, head_scale;
    int64_t num_tokens;
    int32_t num_heads;
    uint32_t heads_mul, heads_shift;
    int32_t scales_word_aligned;  // fp4: every head's group of scale bytes starts on a 4-byte boundary
};

__device__ __forceinline__ float load_weight(const uint8_t* base, int64_t idx, int dtype) {
    if (dtype == 2) return reinterpret_cast<const float*>(base)[idx];
    const uint16_t h = reinterpret_cast<const uint16_t*>(base)[idx];
    if (dtype == 0) return bf16_lo(h);
    float f;
    asm("{.reg .f16 t; mov.b16 t, %1; cvt.f32.f16 %0, t;}" : "=f"(f) : "h"(h));
    return f;
}

// UE8M0 byte of an MXFP4 block whose absolute maximum is `amax`: ceil(log2(max(amax, 6*2^-126) / 6)) + 127 clamped to
// [0, 254], without the division: 6 = 1.5 * 4, so with the clamped maximum m * 2^(E-127), 1 <= m < 2, the quotient is
// below, at or above 2^(E-129) for m below, at or above 1.5.  Equal to the log2/ceil statement for every bf16
// maximum (a CPU test enumerates them).
__device__ __forceinline__ uint32_t mxfp4_code(float amax) {
    const uint32_t u = __float_as_uint(fmaxf(amax, 6.0f * 1.17549435e-38f));
    const uint32_t code = (u >> 23) - 2u + ((u & 0x7fffffu) > 0x400000u ? 1u : 0u);
    return code > 254u ? 254u : code;
}

// Two floats -> one byte of two e2m1 codes (lo in bits 0-3), round to nearest even, saturating at +-6.
__device__ __forceinline__ uint32_t pack_e2m1x2(float lo, float hi) {
    uint32_t r;
    asm("{.reg .b8 t; cvt.rn.satfinite.e2m1x2.f32 t, %1, %2; cvt.u32.u8 %0, t;}" : "=r"(r) : "f"(hi), "f"(lo));
    return r;
}

// Four packed bf16 pairs -> one word of eight e2m1 codes (element 0 in bits 0-3), round to nearest even, saturating at +-6.
__device__ __forceinline__ uint32_t pack_e2m1x8(const uint32_t (&w)[4]) {
    uint32_t r;
    asm("{.reg .b8 t0, t1, t2, t3;\n\t"
        "cvt.rn.satfinite.e2m1x2.f32 t0, %2, %1;\n\t"
        "cvt.rn.satfinite.e2m1x2.f32 t1, %4, %3;\n\t"
        "cvt.rn.satfinite.e2m1x2.f32 t2, %6, %5;\n\t"
        "cvt.rn.satfinite.e2m1x2.f32 t3, %8, %7;\n\t"
        "mov.b32 %0, {t0, t1, t2, t3};}"
        : "=r"(r)
        : "f"(bf16_lo(w[0])), "f"(bf16_hi(w[0])), "f"(bf16_lo(w[1])), "f"(bf16_hi(w[1])), "f"(bf16_lo(w[2])), "f"(bf16_hi(w[2])),
          "f"(bf16_lo(w[3])), "f"(bf16_hi(w[3])));
    return r;
}

// Four packed bf16 pairs times 2^(127 - code): exact (a power-of-two factor only moves the exponent; products below the
// bf16 range become zero with their sign, as their e2m1 codes would anyway).
__device__ __forceinline__ void scale_pow2_bf16x2(const uint32_t (&v)[4], uint32_t code, uint32_t (&w)[4]) {
    const uint32_t inv2 = ((254u - code) << 7) * 0x00010001u;
#pragma unroll
    for (int j = 0; j < 4; ++j) asm("mul.rn.bf16x2 %0, %1, %2;" : "=r"(w[j]) : "r"(v[j]), "r"(inv2));
}

template <int E>
__device__ __forceinline__ void load_row(const uint8_t* p, float (&x)[E]) {
    if (E == 2) {
        const uint32_t v = *reinterpret_cast<const uint32_t*>(p);
        x[0] = bf16_lo(v), x[1] = bf16_hi(v);
    } else if (E == 4) {
        const uint2 v = *reinterpret_cast<const uint2*>(p);
        x[0] = bf16_lo(v.x), x[1] = bf16_hi(v.x), x[2] = bf16_lo(v.y), x[3] = bf16_hi(v.y);
    } else {
        const uint4 v = *reinterpret_cast<const uint4*>(p);
        const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) x[2 * i] = bf16_lo(w[i]), x[2 * i + 1] = bf16_hi(w[i]);
    }
}

template <int WARPS, int E, bool FP4>
__global__ void __launch_bounds__(WARPS * 32) indexer_q_rope_quant_kernel(const IndexerQParams p) {
    constexpr int D = 32 * E;
    const int lane = threadIdx.x & 31;
    const uint32_t row = blockIdx.x * WARPS + (threadIdx.x >> 5);
    if (row >= static_cast<uint32_t>(p.num_tokens) * static_cast<uint32_t>(p.num_heads)) return;
    const uint32_t t = fast_div(row, p.heads_mul, p.heads_shift);
    const int h = static_cast<int>(row - t * static_cast<uint32_t>(p.num_heads));
    float x[E];
    load_row<E>(p.q + (static_cast<int64_t>(t) * p.q_stride0 + h * p.q_stride1 + lane * E) * 2, x);
    const int first_rot = lane * E - (D - p.rot_dim);  // index of this lane's first value inside the rotary tail
    if (first_rot >= 0) {
        const int64_t pos = p.positions[t];
        const int half = p.rot_dim >> 1;
#pragma unroll
        for (int j = 0; j < E / 2; ++j) {
            const int pair = (first_rot >> 1) + j;
            float c, s;
            if (p.cos_sin_bf16) {
                const uint16_t* cs = reinterpret_cast<const uint16_t*>(p.cos_sin) + pos * p.cos_sin_stride;
                c = bf16_lo(cs[pair]), s = bf16_lo(cs[half + pair]);
            } else {
                const float* cs = reinterpret_cast<const float*>(p.cos_sin) + pos * p.cos_sin_stride;
                c = cs[pair], s = cs[half + pair];
            }
            const float e = x[2 * j], o = x[2 * j + 1];
            // separately rounded products, then the bf16 round trip the reference makes before quantising
            const uint32_t packed = pack_bf16x2(__fsub_rn(__fmul_rn(e, c), __fmul_rn(o, s)),
                                                __fadd_rn(__fmul_rn(o, c), __fmul_rn(e, s)));
            x[2 * j] = bf16_lo(packed), x[2 * j + 1] = bf16_hi(packed);
        }
    }
    float amax = 0.0f;
#pragma unroll
    for (int i = 0; i < E; ++i) amax = fmaxf(amax, fabsf(x[i]));
    uint8_t* out = p.out + static_cast<int64_t>(t) * p.out_stride0 + h * p.out_stride1;
    float weight_factor = 1.0f;
    if (FP4) {
        constexpr int kGroupLanes = 32 / E;  // lanes per block of 32 values
#pragma unroll
        for (int m = 1; m < kGroupLanes; m <<= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, m));
        const uint32_t code = mxfp4_code(amax);
        const float inv = __uint_as_float((254u - code) << 23);  // code >= 1 because of the amax floor
        uint32_t bytes = 0;
#pragma unroll
        for (int j = 0; j < E / 2; ++j) bytes |= pack_e2m1x2(__fmul_rn(x[2 * j], inv), __fmul_rn(x[2 * j + 1], inv)) << (8 * j);
        if (E == 2) out[lane] = static_cast<uint8_t>(bytes);
        else if (E == 4) *reinterpret_cast<uint16_t*>(out + 2 * lane) = static_cast<uint16_t>(bytes);
        else *reinterpret_cast<uint32_t*>(out + 4 * lane) = bytes;
        if ((lane & (kGroupLanes - 1)) == 0)
            p.scales[static_cast<int64_t>(t) * p.scale_stride0 + h * p.scale_stride1 + lane / kGroupLanes] = static_cast<uint8_t>(code);
    } else {
#pragma unroll
        for (int m = 16; m > 0; m >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, m));
        const uint32_t code = ue8m0_code(amax);  // 2^ceil(log2(max(amax, 1e-4)/448))
        const float inv = __uint_as_float((254u - code) << 23);
        weight_factor = __uint_as_float(code << 23);
        float y[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int i = 0; i < E; ++i) y[i] = __fmul_rn(x[i], inv);
        if (E == 2) *reinterpret_cast<uint16_t*>(out + 2 * lane) = static_cast<uint16_t>(pack_e4m3x4(y[0], y[1], 0.f, 0.f));
        else if (E == 4) *reinterpret_cast<uint32_t*>(out + 4 * lane) = pack_e4m3x4(y[0], y[1], y[2], y[3]);
        else st_global8(out + 8 * lane, make_uint2(pack_e4m3x4(y[0], y[1], y[2], y[3]), pack_e4m3x4(y[4], y[5], y[6], y[7])));
    }
    if (lane == 0) {
        float w = load_weight(p.weights, static_cast<int64_t>(t) * p.weights_stride + h, p.weights_dtype);
        if (!FP4) w = __fmul_rn(w, weight_factor);
        w = __fmul_rn(__fmul_rn(w, p.softmax_scale), p.head_scale);
        p.weights_out[static_cast<int64_t>(t) * p.weights_out_stride + h] = w;
    }
}

// Fast shape: a row is D/8 lanes holding 8 values (16 bytes) each, so one warp instruction moves 32/G rows;
// U passes per warp are loaded before any is used.  Needs 16-byte aligned rows and a rotary tail that starts
// on a multiple of 8 values.
template <int WARPS, int G, int U, bool FP4>
__global__ void __launch_bounds__(WARPS * 32) indexer_q_rope_quant_rows_kernel(const IndexerQParams p, const int cs_vec4) {
    constexpr int D = 8 * G, ROWS = 32 / G;
    const int lane = threadIdx.x & 31, sub = lane % G, slot = lane / G;
    const uint32_t total = static_cast<uint32_t>(p.num_tokens) * static_cast<uint32_t>(p.num_heads);
    const uint32_t base_row = (blockIdx.x * WARPS + (threadIdx.x >> 5)) * (U * ROWS) + slot;
    uint4 raw[U];
    uint32_t tok[U];
    bool live[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
        const uint32_t row = base_row + u * ROWS;
        live[u] = row < total;
        tok[u] = fast_div(live[u] ? row : 0u, p.heads_mul, p.heads_shift);
        raw[u] = make_uint4(0u, 0u, 0u, 0u);
        if (live[u]) {
            const int h = static_cast<int>(row - tok[u] * static_cast<uint32_t>(p.num_heads));
            raw[u] = ld_stream16(p.q + (static_cast<int64_t>(tok[u]) * p.q_stride0 + h * p.q_stride1 + 8 * sub) * 2);
        }
    }
    const int first_rot = 8 * sub - (D - p.rot_dim);
    const int half = p.rot_dim >> 1;
#pragma unroll
    for (int u = 0; u < U; ++u) {
        const uint32_t row = base_row + u * ROWS;
        const int h = static_cast<int>(row - tok[u] * static_cast<uint32_t>(p.num_heads));
        float x[8];
        unpack8(raw[u], x);
        if (live[u] && first_rot >= 0) {
            const int64_t pos = p.positions[tok[u]];
            const int pair0 = first_rot >> 1;
            float c[4], sn[4];
            if (cs_vec4) {
                const float* cs = reinterpret_cast<const float*>(p.cos_sin) + pos * p.cos_sin_stride;
                const float4 c4 = ld_readonly_f4(cs + pair0), s4 = ld_readonly_f4(cs + half + pair0);
                c[0] = c4.x, c[1] = c4.y, c[2] = c4.z, c[3] = c4.w, sn[0] = s4.x, sn[1] = s4.y, sn[2] = s4.z, sn[3] = s4.w;
            } else if (p.cos_sin_bf16) {
                const uint16_t* cs = reinterpret_cast<const uint16_t*>(p.cos_sin) + pos * p.cos_sin_stride;
#pragma unroll
                for (int j = 0; j < 4; ++j) c[j] = bf16_lo(cs[pair0 + j]), sn[j] = bf16_lo(cs[half + pair0 + j]);
            } else {
                const float* cs = reinterpret_cast<const float*>(p.cos_sin) + pos * p.cos_sin_stride;
#pragma unroll
                for (int j = 0; j < 4; ++j) c[j] = cs[pair0 + j], sn[j] = cs[half + pair0 + j];
            }
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float e = x[2 * j], o = x[2 * j + 1];
                const uint32_t packed = pack_bf16x2(__fsub_rn(__fmul_rn(e, c[j]), __fmul_rn(o, sn[j])),
                                                    __fadd_rn(__fmul_rn(o, c[j]), __fmul_rn(e, sn[j])));
                x[2 * j] = bf16_lo(packed), x[2 * j + 1] = bf16_hi(packed);
            }
        }
        float amax = 0.0f;
#pragma unroll
        for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(x[i]));
        uint8_t* out = p.out + static_cast<int64_t>(tok[u]) * p.out_stride0 + h * p.out_stride1;
        float weight_factor = 1.0f;
        if (FP4) {
#pragma unroll
            for (int m = 1; m < 4; m <<= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, m));
            const uint32_t code = mxfp4_code(amax);
            const float inv = __uint_as_float((254u - code) << 23);
            uint32_t bytes = 0;
#pragma unroll
            for (int j = 0; j < 4; ++j) bytes |= pack_e2m1x2(__fmul_rn(x[2 * j], inv), __fmul_rn(x[2 * j + 1], inv)) << (8 * j);
            if (live[u]) {
                *reinterpret_cast<uint32_t*>(out + 4 * sub) = bytes;
                if ((sub & 3) == 0)
                    p.scales[static_cast<int64_t>(tok[u]) * p.scale_stride0 + h * p.scale_stride1 + (sub >> 2)] = static_cast<uint8_t>(code);
            }
        } else {
#pragma unroll
            for (int m = 1; m < G; m <<= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, m));
            const uint32_t code = ue8m0_code(amax);
            const float inv = __uint_as_float((254u - code) << 23);
            weight_factor = __uint_as_float(code << 23);
#pragma unroll
            for (int i = 0; i < 8; ++i) x[i] = __fmul_rn(x[i], inv);
            if (live[u]) st_global8(out + 8 * sub, make_uint2(pack_e4m3x4(x[0], x[1], x[2], x[3]), pack_e4m3x4(x[4], x[5], x[6], x[7])));
        }
        if (live[u] && sub == 0) {
            float w = load_weight(p.weights, static_cast<int64_t>(tok[u]) * p.weights_stride + h, p.weights_dtype);
            if (!FP4) w = __fmul_rn(w, weight_factor);
            p.weights_out[static_cast<int64_t>(tok[u]) * p.weights_out_stride + h] = __fmul_rn(__fmul_rn(w, p.softmax_scale), p.head_scale);
        }
    }
}

template <int G>
cudaError_t launch_rows(const IndexerQParams& p, bool fp4, int64_t rows, int cs_vec4, cudaStream_t stream) {
    constexpr int WARPS = 4, U = 2, PER_CTA = WARPS * U * (32 / G);
    const unsigned grid = static_cast<unsigned>((rows + PER_CTA - 1) / PER_CTA);
    if (fp4) indexer_q_rope_quant_rows_kernel<WARPS, G, U, true><<<grid, WARPS * 32, 0, stream>>>(p, cs_vec4);
    else indexer_q_rope_quant_rows_kernel<WARPS, G, U, false><<<grid, WARPS * 32, 0, stream>>>(p, cs_vec4);
    return cudaGetLastError();
}

// Large batches of the DeepSeek-V4 geometry (head_dim 128 = 64 un-rotated + 64 rotary): one warp per TOKEN.
// A head is 8 lanes; lane s keeps un-rotated values [8s, 8s+8) and rotary values [64+8s, 64+8s+8) (four pairs), so
// every lane rotates (no divergence), the lane's four cosines and sines are loaded once per token and reused for
// every head, and pointers advance by constants from one group of four heads to the next.  MXFP4 blocks of 32 are
// 4 lanes.
template <int WARPS, bool FP4>
__global__ void __launch_bounds__(WARPS * 32) indexer_q_rope_quant_token_kernel(const IndexerQParams p) {
    const int lane = threadIdx.x & 31, sub = lane & 7, which = lane >> 3;
    const int64_t t = static_cast<int64_t>(blockIdx.x) * WARPS + (threadIdx.x >> 5);
    if (t >= p.num_tokens) return;
    const int64_t pos = p.positions[t];
    float c[4], sn[4];
    if (p.cos_sin_bf16) {
        const uint16_t* cs = reinterpret_cast<const uint16_t*>(p.cos_sin) + pos * p.cos_sin_stride + 4 * sub;
#pragma unroll
        for (int j = 0; j < 4; ++j) c[j] = bf16_lo(cs[j]), sn[j] = bf16_lo(cs[32 + j]);
    } else {
        const float* cs = reinterpret_cast<const float*>(p.cos_sin) + pos * p.cos_sin_stride + 4 * sub;
#pragma unroll
        for (int j = 0; j < 4; ++j) c[j] = cs[j], sn[j] = cs[32 + j];
    }
    const uint8_t* q_tok = p.q + t * p.q_stride0 * 2 + 16 * sub;
    uint8_t* out_tok = p.out + t * p.out_stride0;
#ifndef DSV4_INDEXER_Q_U
#define DSV4_INDEXER_Q_U 2
#endif
    constexpr int U = DSV4_INDEXER_Q_U;  // groups of four heads per pass
    // Two passes are in flight: the loads of the next pass go out before the current one is worked on, so a warp
    // always has rows on their way while it computes.
    uint4 nope[U], rope[U], nope_next[U], rope_next[U];
    const auto load_pass = [&](int h0, uint4 (&n)[U], uint4 (&r)[U]) {
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int h = h0 + 4 * u + which;
            n[u] = r[u] = make_uint4(0u, 0u, 0u, 0u);
            if (h < p.num_heads) {
                const uint8_t* row = q_tok + h * p.q_stride1 * 2;
                n[u] = ld_stream16(row);
                r[u] = ld_stream16(row + 128);
            }
        }
    };
    load_pass(0, nope, rope);
    for (int h0 = 0; h0 < p.num_heads; h0 += 4 * U) {
        load_pass(h0 + 4 * U, nope_next, rope_next);  // past the last head: zeros, nothing is loaded
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int h = h0 + 4 * u + which;
            const bool live = h < p.num_heads;
            float y[8];
            unpack8(rope[u], y);
            uint32_t rot[4];  // the rotated pairs, rounded to bf16 as the reference does before quantising
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float e = y[2 * j], o = y[2 * j + 1];
                // separately rounded products
                rot[j] = pack_bf16x2(__fsub_rn(__fmul_rn(e, c[j]), __fmul_rn(o, sn[j])),
                                     __fadd_rn(__fmul_rn(o, c[j]), __fmul_rn(e, sn[j])));
            }
            uint8_t* out = out_tok + h * p.out_stride1;
            float weight_factor = 1.0f;
            if (FP4) {
                // everything on the packed words: |.| maxima of the un-rotated half (low 16 bits of `both`) and of the
                // rotated half (high 16 bits) reduced together over the 4 lanes of a block of 32
                const uint32_t plain[4] = {nope[u].x, nope[u].y, nope[u].z, nope[u].w};
                const uint32_t pn = max_abs_bf16x2(max_abs_bf16x2(plain[0], plain[1]), max_abs_bf16x2(plain[2], plain[3]));
                const uint32_t pr = max_abs_bf16x2(max_abs_bf16x2(rot[0], rot[1]), max_abs_bf16x2(rot[2], rot[3]));
                uint32_t both = max_abs_bf16x2(__byte_perm(pn, pr, 0x5410), __byte_perm(pn, pr, 0x7632)) & 0x7fff7fffu;
#pragma unroll
                for (int m = 1; m < 4; m <<= 1) both = max_bf16x2(both, __shfl_xor_sync(0xffffffffu, both, m));
                const uint32_t code_n = mxfp4_code(bf16_lo(both)), code_r = mxfp4_code(bf16_hi(both));
                uint32_t wn[4], wr[4];
                scale_pow2_bf16x2(plain, code_n, wn);
                scale_pow2_bf16x2(rot, code_r, wr);
                const uint32_t bn = pack_e2m1x8(wn), br = pack_e2m1x8(wr);
                // the head's four scale bytes in one word: blocks (un-rotated 0-31, 32-63, rotated 0-31, 32-63)
                const uint32_t mine = code_n | (code_r << 16);
                const uint32_t other = __shfl_xor_sync(0xffffffffu, mine, 4);
                if (live) {
                    *reinterpret_cast<uint32_t*>(out + 4 * sub) = bn;
                    *reinterpret_cast<uint32_t*>(out + 32 + 4 * sub) = br;
                    if (sub == 0) {
                        uint8_t* sc = p.scales + t * p.scale_stride0 + h * p.scale_stride1;
                        const uint32_t word = (mine & 0xffu) | ((other & 0xffu) << 8) | (mine & 0xff0000u) | ((other & 0xff0000u) << 8);
                        if (p.scales_word_aligned) {
                            *reinterpret_cast<uint32_t*>(sc) = word;
                        } else {
                            sc[0] = static_cast<uint8_t>(word), sc[1] = static_cast<uint8_t>(word >> 8);
                            sc[2] = static_cast<uint8_t>(word >> 16), sc[3] = static_cast<uint8_t>(word >> 24);
                        }
                    }
                }
            } else {
                float x[8];
                unpack8(nope[u], x);
#pragma unroll
                for (int j = 0; j < 4; ++j) y[2 * j] = bf16_lo(rot[j]), y[2 * j + 1] = bf16_hi(rot[j]);
                float amax = 0.0f;
#pragma unroll
                for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fmaxf(fabsf(x[i]), fabsf(y[i])));
#pragma unroll
                for (int m = 1; m < 8; m <<= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, m));
                const uint32_t code = ue8m0_code(amax);
                const float inv = __uint_as_float((254u - code) << 23);
                weight_factor = __uint_as_float(code << 23);
#pragma unroll
                for (int i = 0; i < 8; ++i) x[i] = __fmul_rn(x[i], inv), y[i] = __fmul_rn(y[i], inv);
                if (live) {
                    st_global8(out + 8 * sub, make_uint2(pack_e4m3x4(x[0], x[1], x[2], x[3]), pack_e4m3x4(x[4], x[5], x[6], x[7])));
                    st_global8(out + 64 + 8 * sub, make_uint2(pack_e4m3x4(y[0], y[1], y[2], y[3]), pack_e4m3x4(y[4], y[5], y[6], y[7])));
                }
            }
            if (live && sub == 0) {
                float w = load_weight(p.weights, t * p.weights_stride + h, p.weights_dtype);
                if (!FP4) w = __fmul_rn(w, weight_factor);
                p.weights_out[t * p.weights_out_stride + h] = __fmul_rn(__fmul_rn(w, p.softmax_scale), p.head_scale);
            }
        }
#pragma unroll
        for (int u = 0; u < U; ++u) nope[u] = nope_next[u], rope[u] = rope_next[u];
    }
}

template <int E>
cudaError_t launch_e(const IndexerQParams& p, bool fp4, unsigned grid, cudaStream_t stream) {
    constexpr int WARPS = 8;
    if (fp4) indexer_q_rope_quant_kernel<WARPS, E, true><<<grid, WARPS * 32, 0, stream>>>(p);
    else indexer_q_rope_quant_kernel<WARPS, E, false><<<grid, WARPS * 32, 0, stream>>>(p);
    return cudaGetLastError();
}

}  // namespace

cudaError_t launch_indexer_q_rope_quant(const int64_t* positions, const void* q, int64_t q_stride0, int64_t q_stride1,
                                        const void* cos_sin, int64_t cos_sin_stride, int cos_sin_bf16, int rot_dim, void* out,
                                        int64_t out_stride0, int64_t out_stride1, void* scales, int64_t scale_stride0,
                                        int64_t scale_stride1, const void* weights, int64_t weights_stride, int weights_dtype,
                                        float* weights_out, int64_t weights_out_stride, float softmax_scale, float head_scale,
                                        int64_t num_tokens, int num_heads, int head_dim, int fp4, cudaStream_t stream) {
    const int64_t rows = num_tokens * num_heads;
    if (rows == 0) return cudaSuccess;
    if (rows >= (1LL << 31)) return cudaErrorInvalidConfiguration;
    IndexerQParams p{};
    p.positions = positions, p.q = static_cast<const uint8_t*>(q), p.q_stride0 = q_stride0, p.q_stride1 = q_stride1;
    p.cos_sin = static_cast<const uint8_t*>(cos_sin), p.cos_sin_stride = cos_sin_stride, p.cos_sin_bf16 = cos_sin_bf16;
    p.rot_dim = rot_dim, p.out = static_cast<uint8_t*>(out), p.out_stride0 = out_stride0, p.out_stride1 = out_stride1;
    p.scales = static_cast<uint8_t*>(scales), p.scale_stride0 = scale_stride0, p.scale_stride1 = scale_stride1;
    p.weights = static_cast<const uint8_t*>(weights), p.weights_stride = weights_stride, p.weights_dtype = weights_dtype;
    p.weights_out = weights_out, p.weights_out_stride = weights_out_stride;
    p.softmax_scale = softmax_scale, p.head_scale = head_scale, p.num_tokens = num_tokens, p.num_heads = num_heads;
    make_fast_divisor(static_cast<uint32_t>(num_heads), &p.heads_mul, &p.heads_shift);
    const auto addr = [](const void* q_) { return reinterpret_cast<uintptr_t>(q_); };
    p.scales_word_aligned = addr(scales) % 4 == 0 && scale_stride0 % 4 == 0 && scale_stride1 % 4 == 0;
    const int nope = head_dim - rot_dim;
    const bool rows_shape = nope % 8 == 0 && rot_dim % 8 == 0 && addr(q) % 16 == 0 && q_stride0 % 8 == 0 && q_stride1 % 8 == 0 &&
                            addr(out) % 8 == 0 && out_stride0 % 8 == 0 && out_stride1 % 8 == 0;
    // one warp per token pays off once there are enough tokens to fill the GPU with warps
    const bool token_shape = head_dim == 128 && rot_dim == 64 && num_tokens >= 8192 && addr(q) % 16 == 0 && q_stride0 % 8 == 0 &&
                             q_stride1 % 8 == 0 && addr(out) % 8 == 0 && out_stride0 % 8 == 0 && out_stride1 % 8 == 0 &&
                             (cos_sin_bf16 || addr(cos_sin) % 4 == 0);
    if (token_shape) {
        constexpr int WARPS = 4;
        const unsigned grid = static_cast<unsigned>((num_tokens + WARPS - 1) / WARPS);
        if (fp4) indexer_q_rope_quant_token_kernel<WARPS, true><<<grid, WARPS * 32, 0, stream>>>(p);
        else indexer_q_rope_quant_token_kernel<WARPS, false><<<grid, WARPS * 32, 0, stream>>>(p);
        count_launch();
        return cudaGetLastError();
    }
    if (rows_shape) {
        const int cs_vec4 = !cos_sin_bf16 && rot_dim > 0 && addr(cos_sin) % 16 == 0 && cos_sin_stride % 4 == 0 && (rot_dim / 2) % 4 == 0;
        cudaError_t e = head_dim == 64 ? launch_rows<8>(p, fp4 != 0, rows, cs_vec4, stream)
                        : head_dim == 128 ? launch_rows<16>(p, fp4 != 0, rows, cs_vec4, stream)
                        : head_dim == 256 ? launch_rows<32>(p, fp4 != 0, rows, cs_vec4, stream) : cudaErrorInvalidValue;
        if (e != cudaErrorInvalidValue) count_launch();
        return e;
    }
    const unsigned grid = static_cast<unsigned>((rows + 7) / 8);
    cudaError_t err;
    if (head_dim == 64) err = launch_e<2>(p, fp4 != 0, grid, stream);
    else if (head_dim == 128) err = launch_e<4>(p, fp4 != 0, grid, stream);
    else if (head_dim == 256) err = launch_e<8>(p, fp4 != 0, grid, stream);
    else return cudaErrorInvalidValue;
    count_launch();
    return err;
}

}  // namespace dsv4
