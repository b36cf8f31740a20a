// Device-side building blocks shared by the prologue kernels (sm_100a only).
//
// Register layouts of one 512-element bf16 row held by one warp.
// "A/B layout" (latent-KV rows):
//   lane i keeps uint4 A = elements [8i, 8i+8)        (bytes 16i .. 16i+15)
//          and  uint4 B = elements [256+8i, 256+8i+8)  (bytes 512+16i ..)
// so each warp-wide 16-byte access covers 512 contiguous bytes, every 64-element
// quantisation group is 8 adjacent lanes of one register (A: groups 0-3, B lanes
// 0-23: groups 4-6) and the 64-element rotary tail [448,512) is B of lanes 24-31,
// whose interleaved (even, odd) pairs are lane-local.
// "A/B/T layout" (q rows): A as above, B only in lanes 0-23 (elements 256..447), and the
// rotary tail as one 4-byte (even, odd) pair per lane: lane j keeps T = elements
// 448+2j, 449+2j.  All 32 lanes then share the rotation work (6 flops each) instead of 8
// lanes doing 4 pairs while 24 wait; accesses stay fully coalesced (512 + 384 + 128 bytes).
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

namespace dsv4 {

constexpr int kHeadDim = 512;
constexpr int kRopeDim = 64;
constexpr int kNopeDim = 448;
constexpr int kRowBytes = kHeadDim * 2;
constexpr int kTokenDataBytes = 576;
constexpr int kScaleBytes = 8;
constexpr int kCosSinRowBytes = 256;
constexpr int kFirstRopeLane = 24;

struct PrologueParams {
    uint8_t* q;             // bf16 [num_tokens, num_heads, 512]
    const uint8_t* kv;      // bf16 [num_tokens, 512]
    uint8_t* k_cache;       // bytes
    const int64_t* slot_mapping;
    const int64_t* position_ids;
    const float* cos_sin;   // fp32 [max_pos, 64]
    float eps;
    int64_t num_tokens;
    int64_t num_heads;
    int64_t num_tokens_insert;
    int64_t block_size;
    int64_t block_stride;   // bytes between cache blocks
    // range checks (checked build only)
    int64_t num_slots;
    int64_t max_pos;
    int32_t* status;
    int cache_aligned16;    // k_cache base and block stride are multiples of 16
    // row / num_heads for row < 2^31 without a divide: (row * heads_mul) >> heads_shift
    uint32_t heads_mul;
    uint32_t heads_shift;
    // out-of-place form only: q rows are written to q_out [num_tokens, out_heads, 512] (out_heads >= num_heads),
    // heads num_heads..out_heads-1 of every token are zero-filled; q itself is then left untouched
    uint8_t* q_out;
    int64_t out_heads;
    // programmatic dependent launch: read position_ids / slot_mapping / cos_sin before the preceding kernel of the
    // stream has finished, wait for it only before touching q and kv (rows variant; 0 = ordinary launch)
    int pdl;
    // rows variant: 1 = the cos|sin rows of a tile go through shared memory (one fetch per CTA), 0 = every warp
    // fetches the table row of its own rows into registers (no barrier; chosen for launches of a few waves)
    int table_staging;
    // bulk variant: SM cycles after which a wait on a shared-memory barrier gives up (the kernel then sets the
    // device error word and returns), and a self-test hook: the tile whose loader announces bytes it never sends
    // (0xffffffff = none)
    long long wait_cycles;
    uint32_t short_tile;
};

// floor(n / d) for n < 2^31 via the multiplier the host derived with make_fast_divisor().
__device__ __forceinline__ uint32_t fast_div(uint32_t n, uint32_t mul, uint32_t shift) {
    return static_cast<uint32_t>((static_cast<uint64_t>(n) * mul) >> shift);
}

// slot -> (block, offset in block); block sizes are powers of two in practice (16, 64): shift and mask then,
// a 64-bit division otherwise.  `shift` < 0 means "not a power of two".
__device__ __forceinline__ void split_slot(int64_t slot, int64_t block_size, int shift, int64_t* block, int64_t* in_block) {
    if (shift >= 0) {
        *block = slot >> shift;
        *in_block = slot & (block_size - 1);
    } else {
        *block = slot / block_size;
        *in_block = slot - *block * block_size;
    }
}

inline int pow2_shift(int64_t v) {
    if (v <= 0 || (v & (v - 1)) != 0) return -1;
    int s = 0;
    while ((1LL << s) < v) ++s;
    return s;
}

// mul = ceil(2^shift / d), shift = 31 + ceil(log2 d): exact for every n < 2^31 and 1 <= d < 2^31,
// because the error d*mul - 2^shift is below d <= 2^(shift-31), so n*error < 2^shift.
inline void make_fast_divisor(uint32_t d, uint32_t* mul, uint32_t* shift) {
    uint32_t l = 0;
    while ((1ull << l) < d) ++l;
    *shift = 31 + l;
    *mul = static_cast<uint32_t>(((1ull << *shift) + d - 1) / d);
}

// ---- memory access ---------------------------------------------------------

// Streaming loads of memory the SAME kernel also writes (q is normalised in place): the ordinary, coherent global
// path, kept out of L1.  The non-coherent path below promises that the data stays read-only while the kernel runs.
__device__ __forceinline__ uint4 ld_inplace16(const void* p) {
    uint4 v;
    asm volatile("ld.global.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}

__device__ __forceinline__ uint32_t ld_inplace4(const void* p) {
    uint32_t v;
    asm volatile("ld.global.L1::no_allocate.u32 %0, [%1];" : "=r"(v) : "l"(p));
    return v;
}

// Streaming 16-byte load of read-only data (never written by the kernel that loads it): touched once, non-coherent
// path, kept out of L1.
__device__ __forceinline__ uint4 ld_stream16(const void* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}

__device__ __forceinline__ void st_stream16(void* p, uint4 v) {
    asm volatile("st.global.L1::no_allocate.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z),
                 "r"(v.w)
                 : "memory");
}

__device__ __forceinline__ uint2 ld_stream8(const void* p) {
    uint2 v;
    asm volatile("ld.global.nc.L1::no_allocate.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p));
    return v;
}

__device__ __forceinline__ uint32_t ld_stream4(const void* p) {
    uint32_t v;
    asm volatile("ld.global.nc.L1::no_allocate.u32 %0, [%1];" : "=r"(v) : "l"(p));
    return v;
}

__device__ __forceinline__ void st_stream4(void* p, uint32_t v) {
    asm volatile("st.global.L1::no_allocate.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

__device__ __forceinline__ void st_global8(void* p, uint2 v) {
    asm volatile("st.global.v2.u32 [%0], {%1,%2};" ::"l"(p), "r"(v.x), "r"(v.y) : "memory");
}

__device__ __forceinline__ float4 ld_readonly_f4(const float* p) {
    return __ldg(reinterpret_cast<const float4*>(p));
}

// ---- number formats --------------------------------------------------------

__device__ __forceinline__ float bf16_lo(uint32_t u) { return __uint_as_float(u << 16); }
__device__ __forceinline__ float bf16_hi(uint32_t u) { return __uint_as_float(u & 0xffff0000u); }

// Two floats -> packed bf16 pair, round to nearest even (lo in bits 0-15).
// Element-wise maximum of two bf16 pairs (one instruction).
__device__ __forceinline__ uint32_t max_bf16x2(uint32_t a, uint32_t b) {
    uint32_t d;
    asm("max.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
    return d;
}

// Element-wise maximum of the magnitudes of two bf16 pairs; the sign bits of the result are the
// exclusive-or of the operands' and carry no meaning (one instruction, no separate absolute value).
__device__ __forceinline__ uint32_t max_abs_bf16x2(uint32_t a, uint32_t b) {
    uint32_t d;
    asm("max.xorsign.abs.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
    return d;
}

__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
    uint32_t r;
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
    return r;
}

// Four floats -> four e4m3 bytes (f0 in the lowest byte), round to nearest even; `satfinite` clamps to
// +-448 (what the reference's explicit clamp before the cast does) and keeps NaN as NaN.
__device__ __forceinline__ uint32_t pack_e4m3x4(float f0, float f1, float f2, float f3) {
    uint16_t lo, hi;
    asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(lo) : "f"(f1), "f"(f0));
    asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(hi) : "f"(f3), "f"(f2));
    return static_cast<uint32_t>(lo) | (static_cast<uint32_t>(hi) << 16);
}

// Two e4m3 bytes (low 16 bits of `pair`) -> two floats, exact.
__device__ __forceinline__ float2 unpack_e4m3x2(uint16_t pair) {
    uint32_t h2;
    asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(h2) : "h"(pair));
    float lo, hi;
    asm("{.reg .f16 l, h; mov.b32 {l, h}, %2; cvt.f32.f16 %0, l; cvt.f32.f16 %1, h;}" : "=f"(lo), "=f"(hi) : "r"(h2));
    return make_float2(lo, hi);
}

__device__ __forceinline__ void unpack8(const uint4& v, float (&x)[8]) {
    x[0] = bf16_lo(v.x), x[1] = bf16_hi(v.x);
    x[2] = bf16_lo(v.y), x[3] = bf16_hi(v.y);
    x[4] = bf16_lo(v.z), x[5] = bf16_hi(v.z);
    x[6] = bf16_lo(v.w), x[7] = bf16_hi(v.w);
}

__device__ __forceinline__ uint4 pack8(const float (&x)[8]) {
    return make_uint4(pack_bf16x2(x[0], x[1]), pack_bf16x2(x[2], x[3]), pack_bf16x2(x[4], x[5]),
                      pack_bf16x2(x[6], x[7]));
}

// ---- q row arithmetic ---------------------------------------------------------

// DSV4_EXACT_SUMSQ=1 accumulates the sum of squares in double, which makes it the correctly
// rounded sum whatever the order (x*x is exact, 512 terms fit double with room to spare), so
// 1/rms equals the CPU oracle's bit for bit when DSV4_IEEE_RSQRT=1 too.  Default 0: fp32 sum
// (the double version costs 6-30 % of the kernel's speed, measured on B200; the fp32 sum moves
// about 1e-5 of the outputs by one bf16 ulp).
#ifndef DSV4_EXACT_SUMSQ
#define DSV4_EXACT_SUMSQ 0
#endif

#if DSV4_EXACT_SUMSQ
typedef double sumsq_t;
#else
typedef float sumsq_t;
#endif

__device__ __forceinline__ sumsq_t sumsq_add8(const float (&x)[8], sumsq_t acc) {
#pragma unroll
    for (int i = 0; i < 8; ++i) {
#if DSV4_EXACT_SUMSQ
        acc = fma(static_cast<double>(x[i]), static_cast<double>(x[i]), acc);
#else
        acc = fmaf(x[i], x[i], acc);
#endif
    }
    return acc;
}

__device__ __forceinline__ sumsq_t warp_sum(sumsq_t v) {
#pragma unroll
    for (int m = 16; m > 0; m >>= 1) v += __shfl_xor_sync(0xffffffffu, v, m);
    return v;
}

// 1/sqrt(mean + eps).  Default: the hardware reciprocal-square-root approximation refined by one
// Newton step (error about 1 fp32 ulp, 6 instructions).  With DSV4_IEEE_RSQRT=1: IEEE square root
// then IEEE division, the two roundings the CPU torch path performs (about 20 instructions).
// The two differ by at most a couple of fp32 ulps, i.e. about 2^-15 of a bf16 ulp: after rounding to bf16
// roughly one output in 10^5 moves by one ulp.  Measured on B200 the IEEE form costs 2 % on large batches.
#ifndef DSV4_IEEE_RSQRT
#define DSV4_IEEE_RSQRT 0
#endif
__device__ __forceinline__ float inv_rms(sumsq_t sum_of_squares, float eps) {
    const float v = __fadd_rn(__fmul_rn(static_cast<float>(sum_of_squares), 1.0f / kHeadDim), eps);
#if DSV4_IEEE_RSQRT
    return __fdiv_rn(1.0f, __fsqrt_rn(v));
#else
    const float r0 = rsqrtf(v);
    const float half_v_r0 = 0.5f * v * r0;
    return fmaf(r0, fmaf(-half_v_r0, r0, 0.5f), r0);  // r0 * (1.5 - 0.5 v r0^2)
#endif
}

// GPT-J rotation of 4 interleaved (even, odd) pairs; c/s are the 4 cosines / sines of
// those pairs.  Products are rounded separately (no FMA) so the result equals the
// reference's `e*c - o*s`, `e*s + o*c` bit for bit.
__device__ __forceinline__ void rotate4(float (&x)[8], const float4& c, const float4& s) {
    const float cc[4] = {c.x, c.y, c.z, c.w};
    const float ss[4] = {s.x, s.y, s.z, s.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const float e = x[2 * j], o = x[2 * j + 1];
        x[2 * j] = __fsub_rn(__fmul_rn(e, cc[j]), __fmul_rn(o, ss[j]));
        x[2 * j + 1] = __fadd_rn(__fmul_rn(e, ss[j]), __fmul_rn(o, cc[j]));
    }
}

// Rotation of the single (even, odd) pair a lane holds in the A/B/T layout; same rounding.
__device__ __forceinline__ uint32_t scale_rotate_pair(uint32_t packed, float r, float c, float s) {
    const float e = __fmul_rn(bf16_lo(packed), r), o = __fmul_rn(bf16_hi(packed), r);
    return pack_bf16x2(__fsub_rn(__fmul_rn(e, c), __fmul_rn(o, s)), __fadd_rn(__fmul_rn(e, s), __fmul_rn(o, c)));
}

__device__ __forceinline__ void scale8(float (&x)[8], float r) {
#pragma unroll
    for (int i = 0; i < 8; ++i) x[i] = __fmul_rn(x[i], r);
}

// One q row in the A/B/T register layout (xb all zero in lanes >= 24): 1/rms of the row, the
// same value in every lane.
__device__ __forceinline__ float row_inv_rms(const float (&xa)[8], const float (&xb)[8], uint32_t tail, float eps) {
    sumsq_t acc = sumsq_add8(xb, sumsq_add8(xa, sumsq_t(0)));
    const float e = bf16_lo(tail), o = bf16_hi(tail);
#if DSV4_EXACT_SUMSQ
    acc = fma(static_cast<double>(o), static_cast<double>(o), fma(static_cast<double>(e), static_cast<double>(e), acc));
#else
    acc = fmaf(o, o, fmaf(e, e, acc));
#endif
    return inv_rms(warp_sum(acc), eps);
}

// ---- UE8M0 quantisation of one 64-element group -----------------------------

// Stored scale byte for a group whose absolute maximum is `amax`:
// clamp(ceil(log2(max(amax, 1e-4) / 448)) + 127, 0, 255), without the division: 448 = 1.75 * 2^8, so with
// a = max(amax, 1e-4) = m * 2^(E-127), 1 <= m < 2, the quotient lies in (2^(E-136), 2^(E-135)) for m < 1.75, is
// exactly 2^(E-135) for m = 1.75 and lies above it for m > 1.75: code = E - 8 + (m > 1.75).  Equal to the
// reference's log2/ceil statement for every bf16 and fp16 amax (their quotients by 448 are exact powers of two
// or at least 0.05 % away from one, so the fp32 rounding of the division cannot cross one); a CPU test checks
// all of them.
__device__ __forceinline__ uint32_t ue8m0_code(float amax) {
    const uint32_t u = __float_as_uint(fmaxf(amax, 1e-4f));
    const uint32_t code = (u >> 23) - 8u + ((u & 0x7fffffu) > 0x600000u ? 1u : 0u);
    return code > 255u ? 255u : code;
}

__device__ __forceinline__ float abs_max8(const uint4& v) {
    float x[8];
    unpack8(v, x);
    float m = 0.0f;
#pragma unroll
    for (int i = 0; i < 8; ++i) m = fmaxf(m, fabsf(x[i]));
    return m;
}

// ---- quantisation with scale = max(amax, eps) / 448 (the epilogue quantiser and the per-token-group quantiser) ----
// Power-of-two scale >= s as (exponent byte, value): ceil(log2(max(s, 1e-10))) from the bit pattern.
__device__ __forceinline__ uint32_t pow2_ceil_code(float s) {
    const uint32_t u = __float_as_uint(fmaxf(s, 1e-10f));
    return ((u >> 23) & 0xffu) + ((u & 0x7fffffu) ? 1u : 0u);
}

// How x / scale is formed for a scale that is not a power of two.
enum : int { kDivideIeee = 0, kDivideFast = 1, kMultiplyReciprocal = 2 };

// kDivideFast: x / scale without an IEEE division.  Once per group: y = the hardware's approximate reciprocal refined
// by one Newton step (relative error about 2^-44 before its rounding, hence within one ulp of RN(1/scale)) and
// y_lo = RN(fma(-scale, y, 1) * y), which brings y + y_lo to about 2^-46 of 1/scale.  Per value, either
//   two-term       q = fma(x, y, RN(x * y_lo))                                    two instructions, scale <= 2^100 only
//                  (beyond that y_lo would be subnormal), or
//   corrected      q0 = RN(x * y), r = fma(-scale, q0, x), q = fma(r, y, q0)      three instructions, any scale.
// q can differ from RN(x/scale) in the last fp32 bit, but never in the e4m3 byte: a CPU test enumerates every bf16
// group maximum (hence every reachable scale, for the reference's eps = 1e-10) against every bf16 value below it, for
// each of the three values y can take (the correctly rounded reciprocal and its two neighbours) and both forms -
// 1.6e9 cases each, zero differing bytes.  The form is a template argument: a caller that uses the two-term form votes once
// per warp on the scales' range (`__all_sync`), so the choice is a uniform branch around straight-line code; the epilogue
// quantiser uses the corrected form throughout (no second code path measured faster there).  For any other eps the
// kernels divide.
// kMultiplyReciprocal: x * RN(1/scale), what the statement of `act_quant` computes.
constexpr float kTwoTermMaxScale = 0x1p100f;

template <int MODE>
struct ScaleDivider {
    float scale, recip, recip_lo;
    __device__ __forceinline__ explicit ScaleDivider(float s) : scale(s), recip(0.0f), recip_lo(0.0f) {
        if (MODE == kMultiplyReciprocal) recip = __frcp_rn(s);
        if (MODE == kDivideFast) {
            float y0;
            asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(y0) : "f"(s));
            recip = __fmaf_rn(__fmaf_rn(-s, y0, 1.0f), y0, y0);
            recip_lo = __fmul_rn(__fmaf_rn(-s, recip, 1.0f), recip);
        }
    }
    __device__ __forceinline__ bool allows_two_term() const { return scale <= kTwoTermMaxScale; }
    // TWO_TERM is honoured in kDivideFast mode only
    template <bool TWO_TERM>
    __device__ __forceinline__ float quotient(float x) const {
        if (MODE == kMultiplyReciprocal) return __fmul_rn(x, recip);
        if (MODE == kDivideIeee) return __fdiv_rn(x, scale);
        if (TWO_TERM) return __fmaf_rn(x, recip, __fmul_rn(x, recip_lo));
        const float q0 = __fmul_rn(x, recip);
        return __fmaf_rn(__fmaf_rn(-scale, q0, x), recip, q0);
    }
};

template <int MODE, bool TWO_TERM>
__device__ __forceinline__ uint2 quant8_by(const uint4& v, const ScaleDivider<MODE>& d) {
    float x[8];
    unpack8(v, x);
    float q[8];  // the e4m3 conversion saturates at +-448
#pragma unroll
    for (int i = 0; i < 8; ++i) q[i] = d.template quotient<TWO_TERM>(x[i]);
    return make_uint2(pack_e4m3x4(q[0], q[1], q[2], q[3]), pack_e4m3x4(q[4], q[5], q[6], q[7]));
}

// 8 bf16 values times the exact reciprocal of a power-of-two scale (same result as dividing by it).  The products are
// formed on the packed words (`mul.rn.bf16x2`: a power-of-two factor only moves the exponent, so bf16 holds them
// exactly; results below the bf16 range become zero with their sign, as their e4m3 bytes would anyway) and widened
// afterwards: 4 multiplies instead of 8.  The reciprocal's exponent field 254 - code is in range for every bf16 maximum.
__device__ __forceinline__ uint2 quant8_pow2(const uint4& v, uint32_t code) {
    const uint32_t inv2 = ((254u - code) << 7) * 0x00010001u;  // 2^(127 - code) in both halves
    uint32_t w[4];
    asm("mul.rn.bf16x2 %0, %1, %2;" : "=r"(w[0]) : "r"(v.x), "r"(inv2));
    asm("mul.rn.bf16x2 %0, %1, %2;" : "=r"(w[1]) : "r"(v.y), "r"(inv2));
    asm("mul.rn.bf16x2 %0, %1, %2;" : "=r"(w[2]) : "r"(v.z), "r"(inv2));
    asm("mul.rn.bf16x2 %0, %1, %2;" : "=r"(w[3]) : "r"(v.w), "r"(inv2));
    return make_uint2(pack_e4m3x4(bf16_lo(w[0]), bf16_hi(w[0]), bf16_lo(w[1]), bf16_hi(w[1])),
                      pack_e4m3x4(bf16_lo(w[2]), bf16_hi(w[2]), bf16_lo(w[3]), bf16_hi(w[3])));
}

// 8 bf16 -> 8 e4m3 bytes of value x / 2^(code-127) (division by a power of two: exact).
__device__ __forceinline__ uint2 quant8(const uint4& v, uint32_t code) {
    const float scale = __uint_as_float(code << 23);
    float x[8];
    unpack8(v, x);
#pragma unroll
    for (int i = 0; i < 8; ++i) x[i] = __fdiv_rn(x[i], scale);
    return make_uint2(pack_e4m3x4(x[0], x[1], x[2], x[3]), pack_e4m3x4(x[4], x[5], x[6], x[7]));
}

// One latent-KV row (A/B layout, registers a,b of this lane) -> its cache slot.
// `data` = first byte of the token's 576-byte record, `scales` = its 8 scale bytes.
// c/s: cosines / sines of this lane's 4 rotary pairs (used by lanes >= 24 only).
__device__ __forceinline__ void kv_row_to_cache(const uint4& a, const uint4& b, int lane, const float4& c,
                                                const float4& s, uint8_t* data, uint8_t* scales, bool aligned16) {
    float ma = abs_max8(a), mb = abs_max8(b);
#pragma unroll
    for (int m = 1; m <= 4; m <<= 1) {
        ma = fmaxf(ma, __shfl_xor_sync(0xffffffffu, ma, m));
        mb = fmaxf(mb, __shfl_xor_sync(0xffffffffu, mb, m));
    }
    const uint32_t code_a = ue8m0_code(ma), code_b = ue8m0_code(mb);
    const uint2 qa = quant8(a, code_a);
    const bool rope_lane = lane >= kFirstRopeLane;
    uint2 qb = make_uint2(0u, 0u);
    uint4 rb = make_uint4(0u, 0u, 0u, 0u);
    if (rope_lane) {
        float x[8];
        unpack8(b, x);
        rotate4(x, c, s);
        rb = pack8(x);
    } else {
        qb = quant8(b, code_b);
    }
    // 7 scale codes + zero pad, assembled in lane 0 (groups 0-3 from A, 4-6 from B)
    uint32_t lo = __shfl_sync(0xffffffffu, code_a, 0) | (__shfl_sync(0xffffffffu, code_a, 8) << 8) |
                  (__shfl_sync(0xffffffffu, code_a, 16) << 16) | (__shfl_sync(0xffffffffu, code_a, 24) << 24);
    uint32_t hi = __shfl_sync(0xffffffffu, code_b, 0) | (__shfl_sync(0xffffffffu, code_b, 8) << 8) |
                  (__shfl_sync(0xffffffffu, code_b, 16) << 16);
    if (aligned16) {
        st_global8(data + 8 * lane, qa);
        if (rope_lane) {
            *reinterpret_cast<uint4*>(data + kNopeDim + 16 * (lane - kFirstRopeLane)) = rb;
        } else {
            st_global8(data + 256 + 8 * lane, qb);
        }
        if (lane == 0) st_global8(scales, make_uint2(lo, hi));
    } else {
        const uint32_t wa[2] = {qa.x, qa.y};
#pragma unroll
        for (int i = 0; i < 8; ++i) data[8 * lane + i] = static_cast<uint8_t>(wa[i >> 2] >> (8 * (i & 3)));
        if (rope_lane) {
            const uint32_t wr[4] = {rb.x, rb.y, rb.z, rb.w};
#pragma unroll
            for (int i = 0; i < 16; ++i)
                data[kNopeDim + 16 * (lane - kFirstRopeLane) + i] = static_cast<uint8_t>(wr[i >> 2] >> (8 * (i & 3)));
        } else {
            const uint32_t wb[2] = {qb.x, qb.y};
#pragma unroll
            for (int i = 0; i < 8; ++i) data[256 + 8 * lane + i] = static_cast<uint8_t>(wb[i >> 2] >> (8 * (i & 3)));
        }
        if (lane < 8) scales[lane] = static_cast<uint8_t>((lane < 4 ? lo : hi) >> (8 * (lane & 3)));
    }
}

// Launchers implemented by the kernel files; each returns cudaGetLastError() of its launch.
cudaError_t launch_prologue_rows(const PrologueParams& p, bool checked, cudaStream_t stream);
cudaError_t launch_prologue_rows_padded(const PrologueParams& p, cudaStream_t stream);
cudaError_t launch_prologue_bulk(const PrologueParams& p, cudaStream_t stream);
cudaError_t launch_gather_dequant(const uint8_t* k_cache, const int64_t* slots, int64_t num_slots, uint8_t* out,
                                  int64_t out_row_stride, int64_t block_size, int64_t block_stride,
                                  cudaStream_t stream);
cudaError_t launch_gather_dequant_requests(uint8_t* out, int64_t out_stride0, int64_t out_stride1, const uint8_t* k_cache,
                                           const void* seq_lens, const void* gather_lens, const void* block_table,
                                           int64_t num_reqs, int64_t max_blocks_per_seq, int64_t block_size,
                                           int64_t block_stride, int64_t offset, int nope_dim, int rope_dim, int scale_slots,
                                           int index64, int64_t tokens_hint, cudaStream_t stream);
cudaError_t launch_q_kv_rmsnorm(const void* q, void* q_out, const void* q_weight, int64_t q_in_stride, int64_t q_out_stride,
                                int64_t q_size, const void* kv, void* kv_out, const void* kv_weight, int64_t kv_in_stride,
                                int64_t kv_out_stride, int64_t kv_size, int64_t num_tokens, float eps, cudaStream_t stream);
cudaError_t launch_inv_rope_fp8_quant(const void* o, int64_t o_stride_token, int64_t o_stride_head, const int64_t* positions,
                                      const float* cos_sin, int64_t cos_sin_stride, void* fp8, void* scale,
                                      int64_t scale_stride_group, int64_t num_tokens, int64_t padded_tokens, int num_heads,
                                      int heads_per_group, float eps, int packed, cudaStream_t stream);
cudaError_t launch_indexer_k_quant(const void* k, int64_t k_stride, int is_fp16, void* cache, int64_t block_stride,
                                   const int64_t* slot_mapping, int64_t num_tokens, int64_t block_size, int head_dim,
                                   int quant_block, int ue8m0, cudaStream_t stream);
cudaError_t launch_cp_gather_indexer(const void* cache, int64_t block_stride, void* k_out, int64_t k_out_stride, void* scale_out,
                                     int64_t scale_out_stride, const int32_t* block_table, int64_t block_table_stride,
                                     const int32_t* cu_seqlen, int64_t batch, int64_t num_tokens, int64_t block_size, int head_dim,
                                     int num_quant_blocks, cudaStream_t stream);
cudaError_t launch_global_topk(const int32_t* local, int64_t local_stride, const int32_t* token_to_req, const int32_t* block_table,
                               int64_t block_table_stride, const int32_t* is_valid, int32_t* global, int64_t global_stride,
                               int32_t* lens, int64_t num_tokens, int topk, int block_size, cudaStream_t stream);
cudaError_t launch_combine_topk_swa(const int32_t* topk_indices, int64_t topk_stride, int topk_width, const int32_t* query_start_loc,
                                    const int32_t* seq_lens, const int32_t* gather_lens, int32_t* combined, int64_t combined_stride,
                                    int combined_width, int32_t* lens, int64_t num_reqs, int64_t num_tokens, int window,
                                    int compress_ratio, int top_k, int m, int n, cudaStream_t stream);
cudaError_t launch_topk_per_row(const float* logits, int64_t stride0, int64_t stride1, int32_t* indices, int64_t num_rows, int vocab,
                                int top_k, const int32_t* seq_lens, int next_n, const int32_t* row_starts, const int32_t* row_ends,
                                cudaStream_t stream);
cudaError_t launch_topk_per_row_short(const float* logits, int64_t stride0, int64_t stride1, int32_t* indices, int64_t num_rows, int vocab,
                                int top_k, const int32_t* seq_lens, int next_n, const int32_t* row_starts, const int32_t* row_ends,
                                cudaStream_t stream);  // 256 threads per CTA: rows up to 8192 wide
cudaError_t launch_group_quant_fp8(const void* x, int64_t x_stride, void* out, float* scales, int64_t scale_stride_row,
                                   int64_t scale_stride_group, int64_t num_rows, int64_t num_cols, int group_size, float eps, int ue8m0,
                                   int act_quant_rules, cudaStream_t stream);
cudaError_t launch_indexer_q_rope_quant(const int64_t* positions, const void* q, int64_t q_stride0, int64_t q_stride1,
                                        const void* cos_sin, int64_t cos_sin_stride, int cos_sin_bf16, int rot_dim, void* out,
                                        int64_t out_stride0, int64_t out_stride1, void* scales, int64_t scale_stride0,
                                        int64_t scale_stride1, const void* weights, int64_t weights_stride, int weights_dtype,
                                        float* weights_out, int64_t weights_out_stride, float softmax_scale, float head_scale,
                                        int64_t num_tokens, int num_heads, int head_dim, int fp4, cudaStream_t stream);
cudaError_t launch_q_kv_rmsnorm_any(const void* q, void* q_out, const void* q_weight, int64_t q_in_stride, int64_t q_out_stride,
                                    int64_t q_size, int q_dtype, int q_weight_dtype, const void* kv, void* kv_out,
                                    const void* kv_weight, int64_t kv_in_stride, int64_t kv_out_stride, int64_t kv_size,
                                    int kv_dtype, int kv_weight_dtype, int64_t num_tokens, float eps, cudaStream_t stream);
cudaError_t launch_inv_rope_fp8_quant_any(const void* o, int64_t o_stride_token, int64_t o_stride_head, const int64_t* positions,
                                          const float* cos_sin, int64_t cos_sin_stride, void* fp8, void* scale,
                                          int64_t scale_stride_group, int64_t num_tokens, int64_t padded_tokens, int num_heads,
                                          int heads_per_group, int nope_dim, int rope_dim, int group_size, float eps, int packed,
                                          cudaStream_t stream);
cudaError_t launch_prologue_rows_any_alignment(const PrologueParams& p, cudaStream_t stream);
void count_launch();
cudaError_t read_device_error(int* value);

}  // namespace dsv4
