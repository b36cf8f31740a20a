/*
 * CPU oracle for the DeepSeek-V4 attention prologue
 * (fused_deepseek_v4_qnorm_rope_kv_rope_quant_insert) and for the reader of the
 * cache rows it writes.
 *
 * TEST INFRASTRUCTURE ONLY.  Nothing in the shipped package may link, load or
 * call this file: it exists so that tests, the smoke check and the benchmark's
 * CPU-baseline leg have an independent statement of the arithmetic to compare
 * the CUDA kernels with.  It is a plain-C restatement of the torch reference
 * path that the upstream project keeps inside its own test file
 * (tests/test_fused_deepseek_v4_qnorm_rope_kv_rope_quant_insert.py); each
 * function cites the lines it follows.  Parity is pinned: the Python test-suite
 * checks this file against golden vectors produced by running that upstream
 * torch path itself (tests/golden/make_golden.py).
 *
 * Build: see oracle/Makefile (must keep -ffp-contract=off: the reference rounds
 * every product separately, an FMA would change results).
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

enum {
    HEAD_DIM = 512,
    ROPE_DIM = 64,
    NOPE_DIM = 448,
    HALF_ROPE = 32,
    QUANT_GROUP = 64,
    NUM_GROUPS = 7,
    SCALE_BYTES = 8,       /* 7 UE8M0 codes + 1 zero pad byte per cached token */
    TOKEN_DATA_BYTES = 576 /* 448 e4m3 bytes + 64 bf16 */
};

/* ---- scalar conversions ------------------------------------------------ */

static inline float bf16_bits_to_f32(uint16_t h) {
    uint32_t u = (uint32_t)h << 16;
    float f;
    memcpy(&f, &u, 4);
    return f;
}

/* float -> bfloat16, round to nearest even (what Tensor.to(torch.bfloat16) does). */
static inline uint16_t f32_to_bf16_bits(float f) {
    uint32_t u;
    memcpy(&u, &f, 4);
    if ((u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((u >> 16) | 0x0040u); /* quiet NaN */
    uint32_t lsb = (u >> 16) & 1u;
    u += 0x7fffu + lsb;
    return (uint16_t)(u >> 16);
}

/*
 * float -> float8_e4m3fn bit pattern, round to nearest even, subnormals kept
 * (the conversion of T:166-175, `x.to(torch.float8_e4m3fn).view(torch.uint8)`).
 * Format: 1 sign, 4 exponent (bias 7), 3 mantissa; no infinities; 0x7f is NaN;
 * largest finite 448 = 0x7e; smallest normal 2^-6; subnormal step 2^-9.
 * Written out from the format definition; pinned against torch in the tests.
 */
static inline uint8_t f32_to_e4m3_bits(float f) {
    uint32_t u;
    memcpy(&u, &f, 4);
    uint8_t sign = (uint8_t)((u >> 24) & 0x80u);
    uint32_t a = u & 0x7fffffffu;
    if (a > 0x7f800000u) return (uint8_t)(sign | 0x7fu); /* NaN */
    float af;
    memcpy(&af, &a, 4);
    uint32_t code;
    if (af < 0.015625f) { /* below 2^-6: count subnormal steps of 2^-9 */
        float steps = nearbyintf(af * 512.0f); /* ties to even under the default mode */
        code = (uint32_t)steps;                /* 0..8; 8 is the smallest normal */
    } else {
        int32_t e = (int32_t)(a >> 23) - 127; /* unbiased exponent, >= -6 here */
        uint32_t frac = a & 0x7fffffu;
        uint32_t m = frac >> 20;
        uint32_t rest = frac & 0xfffffu;
        if (rest > 0x80000u || (rest == 0x80000u && (m & 1u))) m++;
        if (m == 8u) {
            m = 0;
            e++;
        }
        if (e > 8) return (uint8_t)(sign | 0x7fu);
        code = ((uint32_t)(e + 7) << 3) | m;
        if (code > 0x7fu) code = 0x7fu; /* rounded past 448: the NaN pattern, as torch */
    }
    return (uint8_t)(sign | code);
}

static inline float e4m3_bits_to_f32(uint8_t b) {
    uint32_t e = (b >> 3) & 0xfu, m = b & 7u;
    float v;
    if (e == 0xfu && m == 7u) return NAN;
    if (e == 0) v = (float)m * 0.001953125f; /* m * 2^-9 */
    else v = ldexpf(1.0f + (float)m * 0.125f, (int)e - 7);
    return (b & 0x80u) ? -v : v;
}

/*
 * UE8M0 scale of one 64-element quant group, the way the reference states it
 * (T:217-223 and T:236-237): exponent = ceil(log2(max(amax,1e-4)/448)),
 * stored code = clamp(exponent+127, 0, 255), scale = 2^(code-127) built from bits
 * (T:154-163).
 */
static inline int ue8m0_exponent_logpath(float amax) {
    float block_max = amax < 1e-4f ? 1e-4f : amax;
    float raw = block_max / 448.0f;
    return (int)ceilf(log2f(raw));
}

/*
 * The same exponent without log or division, the derivation the CUDA kernels use: 448 = 1.75 * 2^8, so with
 * max(amax, 1e-4) = m * 2^e (1 <= m < 2) the exponent is e - 8, plus one when m > 1.75.  The tests prove it
 * equal to the log path for every bf16 and fp16 amax.
 */
static inline int ue8m0_exponent_bitpath(float amax) {
    float block_max = amax < 1e-4f ? 1e-4f : amax;
    uint32_t u;
    memcpy(&u, &block_max, 4);
    return (int)(u >> 23) - 127 - 8 + ((u & 0x7fffffu) > 0x600000u ? 1 : 0);
}

static inline float pow2_from_code(int code) {
    uint32_t u = (uint32_t)code << 23;
    float f;
    memcpy(&f, &u, 4);
    return f;
}

static inline int clampi(int v, int lo, int hi) { return v < lo ? lo : (v > hi ? hi : v); }

/* ---- exported scalar probes (used by the tests to pin the conversions) --- */

void dsv4_oracle_bf16_from_f32(const float* src, uint16_t* dst, int64_t n) {
    for (int64_t i = 0; i < n; ++i) dst[i] = f32_to_bf16_bits(src[i]);
}

void dsv4_oracle_e4m3_from_f32(const float* src, uint8_t* dst, int64_t n) {
    for (int64_t i = 0; i < n; ++i) dst[i] = f32_to_e4m3_bits(src[i]);
}

void dsv4_oracle_f32_from_e4m3(const uint8_t* src, float* dst, int64_t n) {
    for (int64_t i = 0; i < n; ++i) dst[i] = e4m3_bits_to_f32(src[i]);
}

/* codes_log / codes_bits: stored UE8M0 byte for each amax, by both derivations. */
void dsv4_oracle_ue8m0_codes(const float* amax, uint8_t* codes_log, uint8_t* codes_bits, int64_t n) {
    for (int64_t i = 0; i < n; ++i) {
        codes_log[i] = (uint8_t)clampi(ue8m0_exponent_logpath(amax[i]) + 127, 0, 255);
        codes_bits[i] = (uint8_t)clampi(ue8m0_exponent_bitpath(amax[i]) + 127, 0, 255);
    }
}

/* ---- the path ----------------------------------------------------------- */

/*
 * GPT-J (interleaved pair) rotation of a 64-float tail, T:93-140: pair j is
 * elements (2j, 2j+1); cs row = 32 cos then 32 sin.  Two rounded products, then
 * one rounded add or subtract.
 */
static inline void rope_tail(float* tail, const float* cs) {
    for (int j = 0; j < HALF_ROPE; ++j) {
        float e = tail[2 * j], o = tail[2 * j + 1];
        float c = cs[j], s = cs[HALF_ROPE + j];
        float ec = e * c, os = o * s, es = e * s, oc = o * c;
        tail[2 * j] = ec - os;
        tail[2 * j + 1] = es + oc;
    }
}

/* One query row in place: weight-less RMSNorm in fp32 (T:143-148), rotate the
 * tail, round everything to bf16 (T:137-140). */
static void q_row(uint16_t* row, const float* cs, float eps) {
    float x[HEAD_DIM];
    double acc = 0.0; /* correctly rounded sum: the centre of every fp32 summation order */
    for (int i = 0; i < HEAD_DIM; ++i) {
        x[i] = bf16_bits_to_f32(row[i]);
        acc += (double)x[i] * (double)x[i];
    }
    float variance = (float)acc / (float)HEAD_DIM;
    float r = 1.0f / sqrtf(variance + eps);
    for (int i = 0; i < HEAD_DIM; ++i) x[i] = x[i] * r;
    rope_tail(x + NOPE_DIM, cs);
    for (int i = 0; i < HEAD_DIM; ++i) row[i] = f32_to_bf16_bits(x[i]);
}

/* One latent KV row into its cache slot, T:178-243 (+ rotation of the raw tail,
 * T:328-333).  `kv_row` is not written. */
static void kv_row_insert(const uint16_t* kv_row, const float* cs, uint8_t* k_cache, int64_t slot,
                          int64_t block_size, int64_t block_stride) {
    int64_t block = slot / block_size, pos = slot % block_size;
    uint8_t* block_base = k_cache + block * block_stride;
    uint8_t* data = block_base + pos * TOKEN_DATA_BYTES;
    uint8_t* scales = block_base + block_size * TOKEN_DATA_BYTES + pos * SCALE_BYTES;

    float tail[ROPE_DIM];
    for (int i = 0; i < ROPE_DIM; ++i) tail[i] = bf16_bits_to_f32(kv_row[NOPE_DIM + i]);
    rope_tail(tail, cs);
    for (int i = 0; i < ROPE_DIM; ++i) {
        uint16_t b = f32_to_bf16_bits(tail[i]);
        memcpy(data + NOPE_DIM + 2 * i, &b, 2);
    }
    for (int g = 0; g < NUM_GROUPS; ++g) {
        float v[QUANT_GROUP], amax = 0.0f;
        for (int i = 0; i < QUANT_GROUP; ++i) {
            v[i] = bf16_bits_to_f32(kv_row[g * QUANT_GROUP + i]);
            float a = fabsf(v[i]);
            if (a > amax || a != a) amax = a; /* NaN sticks, like torch.max */
        }
        int exponent = ue8m0_exponent_logpath(amax);
        int code = clampi(exponent + 127, 0, 255);
        float scale = pow2_from_code(code);
        for (int i = 0; i < QUANT_GROUP; ++i) {
            float t = v[i] / scale;
            if (t < -448.0f) t = -448.0f;
            if (t > 448.0f) t = 448.0f;
            data[g * QUANT_GROUP + i] = f32_to_e4m3_bits(t);
        }
        scales[g] = (uint8_t)code;
    }
    scales[NUM_GROUPS] = 0;
}

/*
 * The whole op on host memory, same argument meaning as the reference's entry
 * point (src/flaggems_vllm/ops/fused_deepseek_v4_qnorm_rope_kv_rope_quant_insert.py:289-351)
 * and the same result as its oracle `ref_impl` (T:316-333) — except that kv is
 * left untouched, as the operator's contract says (the upstream oracle rotates
 * its private copy).  q [N,H,512] bf16 in place; kv [N,512] bf16; k_cache bytes
 * with `block_stride` bytes per block; slot_mapping [n_insert] (entries < 0
 * skipped; tokens >= n_insert never inserted); position_ids [N]; cos_sin
 * [max_pos,64] fp32.  Returns 0, or -1 on a negative size.
 */
int dsv4_oracle_prologue(uint16_t* q, const uint16_t* kv, uint8_t* k_cache, const int64_t* slot_mapping,
                         const int64_t* position_ids, const float* cos_sin, float eps, int64_t num_tokens,
                         int64_t num_heads, int64_t num_tokens_insert, int64_t block_size, int64_t block_stride,
                         int num_threads) {
    if (num_tokens < 0 || num_heads < 0 || num_tokens_insert < 0 || num_tokens_insert > num_tokens) return -1;
#ifdef _OPENMP
    if (num_threads > 0) omp_set_num_threads(num_threads);
#else
    (void)num_threads;
#endif
#pragma omp parallel for schedule(static)
    for (int64_t t = 0; t < num_tokens; ++t) {
        const float* cs = cos_sin + position_ids[t] * ROPE_DIM;
        for (int64_t h = 0; h < num_heads; ++h) q_row(q + (t * num_heads + h) * HEAD_DIM, cs, eps);
        if (t < num_tokens_insert && slot_mapping[t] >= 0)
            kv_row_insert(kv + t * HEAD_DIM, cs, k_cache, slot_mapping[t], block_size, block_stride);
    }
    return 0;
}

/*
 * Reader of the rows written above: out[i,:] for i < n_slots is the bf16
 * de-quantised token stored at slots[i] — 448 values e4m3 * 2^(code-127) rounded
 * to bf16, then the 64 bf16 RoPE values copied.  Follows the arithmetic of
 * src/flaggems_vllm/ops/deepseek_v4_attention_dequantize_and_gather_k_cache.py:86-120
 * (value = e4m3 * exp2(code - 127); RoPE part copied).  A slot < 0 yields a zero row.
 */
int dsv4_oracle_gather_dequant(const uint8_t* k_cache, const int64_t* slots, int64_t n_slots, uint16_t* out,
                               int64_t block_size, int64_t block_stride, int num_threads) {
    if (n_slots < 0) return -1;
#ifdef _OPENMP
    if (num_threads > 0) omp_set_num_threads(num_threads);
#else
    (void)num_threads;
#endif
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < n_slots; ++i) {
        uint16_t* row = out + i * HEAD_DIM;
        int64_t slot = slots[i];
        if (slot < 0) {
            memset(row, 0, HEAD_DIM * 2);
            continue;
        }
        int64_t block = slot / block_size, pos = slot % block_size;
        const uint8_t* block_base = k_cache + block * block_stride;
        const uint8_t* data = block_base + pos * TOKEN_DATA_BYTES;
        const uint8_t* scales = block_base + block_size * TOKEN_DATA_BYTES + pos * SCALE_BYTES;
        for (int g = 0; g < NUM_GROUPS; ++g) {
            float scale = exp2f((float)scales[g] - 127.0f);
            for (int j = 0; j < QUANT_GROUP; ++j)
                row[g * QUANT_GROUP + j] = f32_to_bf16_bits(e4m3_bits_to_f32(data[g * QUANT_GROUP + j]) * scale);
        }
        memcpy(row + NOPE_DIM, data + NOPE_DIM, ROPE_DIM * 2);
    }
    return 0;
}

/*
 * The request / block-table form of the reader, any nope / rope / scale_slots:
 * src/flaggems_vllm/ops/deepseek_v4_attention_dequantize_and_gather_k_cache.py:61-120.
 * out[r, offset+i, :] for i < gather_lens[r] (seq_lens[r] when gather_lens is NULL) is the token at
 * position seq_lens[r]-gather_len+i of request r; int32 index arrays; out strides in elements.
 */
int dsv4_oracle_dequantize_and_gather(uint16_t* out, int64_t stride0, int64_t stride1, const uint8_t* k_cache,
                                      const int32_t* seq_lens, const int32_t* gather_lens, const int32_t* block_table,
                                      int64_t num_reqs, int64_t max_blocks_per_seq, int64_t block_size,
                                      int64_t block_stride, int64_t offset, int nope_dim, int rope_dim, int scale_slots) {
    if (num_reqs < 0 || nope_dim < 0 || rope_dim < 0) return -1;
    const int64_t token_data = nope_dim + 2 * rope_dim;
    for (int64_t r = 0; r < num_reqs; ++r) {
        int64_t seq_len = seq_lens[r], gather_len = gather_lens ? gather_lens[r] : seq_len;
        for (int64_t i = 0; i < gather_len; ++i) {
            int64_t pos = seq_len - gather_len + i;
            int64_t block = block_table[r * max_blocks_per_seq + pos / block_size], in_block = pos % block_size;
            const uint8_t* base = k_cache + block * block_stride;
            const uint8_t* data = base + in_block * token_data;
            const uint8_t* scales = base + block_size * token_data + in_block * scale_slots;
            uint16_t* row = out + r * stride0 + (offset + i) * stride1;
            for (int j = 0; j < nope_dim; ++j)
                row[j] = f32_to_bf16_bits(e4m3_bits_to_f32(data[j]) * exp2f((float)scales[j / 64] - 127.0f));
            memcpy(row + nope_dim, data + nope_dim, (size_t)rope_dim * 2);
        }
    }
    return 0;
}

/*
 * Weighted RMSNorm of `rows` rows of `size` bf16 values: out = (x * rsqrt(mean(x^2) + eps)) * w, the
 * statement of tests/test_deepseek_v4_attention_fused_q_kv_rmsnorm.py:40-44 (`_rmsnorm_ref`) and of
 * src/flaggems_vllm/ops/deepseek_v4_attention_fused_q_kv_rmsnorm.py:55-61.  Strides in elements.
 */
int dsv4_oracle_weighted_rmsnorm(const uint16_t* x, const uint16_t* w, uint16_t* out, int64_t rows, int64_t size,
                                 int64_t in_stride, int64_t out_stride, float eps) {
    if (rows < 0 || size <= 0) return -1;
    for (int64_t r = 0; r < rows; ++r) {
        const uint16_t* xi = x + r * in_stride;
        double acc = 0.0;
        for (int64_t i = 0; i < size; ++i) {
            double v = bf16_bits_to_f32(xi[i]);
            acc += v * v;
        }
        float variance = (float)acc / (float)size;
        float rr = 1.0f / sqrtf(variance + eps);
        for (int64_t i = 0; i < size; ++i) {
            float y = bf16_bits_to_f32(xi[i]) * rr;
            out[r * out_stride + i] = f32_to_bf16_bits(y * bf16_bits_to_f32(w[i]));
        }
    }
    return 0;
}

/*
 * Inverse GPT-J RoPE + FP8 quantisation in groups of `group` values of o [N, H, nope_dim + rope_dim]
 * (H = n_groups*heads_per_group; the rotary tail ends the last group), the torch statement
 * tests/test_fused_inv_rope_fp8_quant.py:132-198 of src/flaggems_vllm/ops/fused_inv_rope_fp8_quant.py:37-152.
 * With K = head_dim / group groups per head:
 * fp8 out: dense [N, n_groups, heads_per_group*head_dim] bytes.  scales out: dense [N, n_groups, .]:
 * fp32 with heads_per_group*K columns, or (packed != 0, K <= 4) int32 with heads_per_group columns, byte j = exponent
 * byte of the power-of-two scale of the head's group j.  o strides in elements.
 */
int dsv4_oracle_inv_rope_fp8_quant_geometry(const uint16_t* o, int64_t stride_token, int64_t stride_head, const int64_t* positions,
                                            const float* cos_sin, int64_t cos_sin_stride, uint8_t* fp8, void* scales,
                                            int64_t num_tokens, int64_t n_groups, int64_t heads_per_group, int64_t nope_dim,
                                            int64_t rope_dim, int64_t group, float eps, int packed) {
    const int64_t head_dim = nope_dim + rope_dim;
    if (num_tokens < 0 || n_groups <= 0 || heads_per_group <= 0 || nope_dim < 0 || rope_dim < 0 || rope_dim % 2 != 0 || group <= 0 ||
        head_dim <= 0 || head_dim > 65536 || head_dim % group != 0 || nope_dim % group != group - rope_dim)
        return -1;
    const int64_t chunks = head_dim / group, half_rope = rope_dim / 2;
    if (packed && chunks > 4) return -1;
    const int64_t heads = n_groups * heads_per_group;
    const float inv_fp8_max = (float)(1.0 / 448.0);
#pragma omp parallel for schedule(static)
    for (int64_t t = 0; t < num_tokens; ++t) {
        const float* cs = cos_sin + positions[t] * cos_sin_stride;
        float* x = (float*)malloc(sizeof(float) * (size_t)head_dim);
        for (int64_t h = 0; h < heads; ++h) {
            const uint16_t* row = o + t * stride_token + h * stride_head;
            for (int64_t i = 0; i < nope_dim; ++i) x[i] = bf16_bits_to_f32(row[i]);
            for (int64_t j = 0; j < half_rope; ++j) {
                float e = bf16_bits_to_f32(row[nope_dim + 2 * j]), od = bf16_bits_to_f32(row[nope_dim + 2 * j + 1]);
                float c = cs[j], sn = cs[half_rope + j];
                float ec = e * c, os = od * sn, oc = od * c, es = e * sn;
                x[nope_dim + 2 * j] = bf16_bits_to_f32(f32_to_bf16_bits(ec + os));
                x[nope_dim + 2 * j + 1] = bf16_bits_to_f32(f32_to_bf16_bits(oc - es));
            }
            int64_t g = h / heads_per_group, hig = h % heads_per_group;
            uint8_t* out = fp8 + ((t * n_groups + g) * heads_per_group + hig) * head_dim;
            uint32_t word = 0;
            for (int64_t k = 0; k < chunks; ++k) {
                float amax = 0.0f;
                for (int64_t i = 0; i < group; ++i) {
                    float a = fabsf(x[group * k + i]);
                    if (a > amax) amax = a;
                }
                float scale = (amax < eps ? eps : amax) * inv_fp8_max;
                if (packed) {
                    float clamped = scale < 1e-10f ? 1e-10f : scale;
                    scale = exp2f(ceilf(log2f(clamped)));
                    uint32_t bits;
                    memcpy(&bits, &scale, 4);
                    word |= ((bits >> 23) & 0xffu) << (8 * k);
                } else {
                    ((float*)scales)[((t * n_groups + g) * heads_per_group + hig) * chunks + k] = scale;
                }
                for (int64_t i = 0; i < group; ++i) {
                    float q = x[group * k + i] / scale;
                    if (q < -448.0f) q = -448.0f;
                    if (q > 448.0f) q = 448.0f;
                    out[group * k + i] = f32_to_e4m3_bits(q);
                }
            }
            if (packed) ((uint32_t*)scales)[(t * n_groups + g) * heads_per_group + hig] = word;
        }
        free(x);
    }
    return 0;
}

/* The DeepSeek-V4 geometry of the function above: head_dim 512 = 448 + 64, groups of 128. */
int dsv4_oracle_inv_rope_fp8_quant(const uint16_t* o, int64_t stride_token, int64_t stride_head, const int64_t* positions,
                                   const float* cos_sin, int64_t cos_sin_stride, uint8_t* fp8, void* scales,
                                   int64_t num_tokens, int64_t n_groups, int64_t heads_per_group, float eps, int packed) {
    return dsv4_oracle_inv_rope_fp8_quant_geometry(o, stride_token, stride_head, positions, cos_sin, cos_sin_stride, fp8, scales,
                                                   num_tokens, n_groups, heads_per_group, NOPE_DIM, ROPE_DIM, 128, eps, packed);
}

static inline float fp16_bits_to_f32(uint16_t h) {
    uint32_t sign = (uint32_t)(h & 0x8000u) << 16, e = (h >> 10) & 0x1fu, m = h & 0x3ffu;
    float v;
    if (e == 0) v = ldexpf((float)m, -24);
    else if (e == 31) v = m ? NAN : INFINITY;
    else v = ldexpf((float)(m | 0x400u), (int)e - 25);
    uint32_t u;
    memcpy(&u, &v, 4);
    u |= sign;
    memcpy(&v, &u, 4);
    return v;
}

/*
 * Sparse-indexer key quantisation into its paged cache, the torch statement
 * tests/test_indexer_k_quant_and_cache.py:99-143 of src/flaggems_vllm/ops/indexer_k_quant_and_cache.py:44-100.
 * k [num_tokens, head_dim] bf16 (fp16 when is_fp16), row stride in elements; cache block b at b*block_stride bytes:
 * block_size*head_dim e4m3 bytes then block_size*(head_dim/quant_block) fp32 scales.
 */
int dsv4_oracle_indexer_k_quant(const uint16_t* k, int64_t k_stride, int is_fp16, uint8_t* cache, int64_t block_stride,
                                const int64_t* slot_mapping, int64_t num_tokens, int64_t block_size, int64_t head_dim,
                                int64_t quant_block, int ue8m0) {
    if (num_tokens < 0 || quant_block <= 0 || head_dim % quant_block != 0) return -1;
    const int64_t nqb = head_dim / quant_block;
    for (int64_t t = 0; t < num_tokens; ++t) {
        int64_t slot = slot_mapping[t];
        if (slot < 0) continue;
        int64_t block = slot / block_size, in_block = slot % block_size;
        uint8_t* base = cache + block * block_stride;
        for (int64_t g = 0; g < nqb; ++g) {
            float amax = 0.0f;
            for (int64_t i = 0; i < quant_block; ++i) {
                uint16_t h = k[t * k_stride + g * quant_block + i];
                float a = fabsf(is_fp16 ? fp16_bits_to_f32(h) : bf16_bits_to_f32(h));
                if (a > amax) amax = a;
            }
            float scale = (amax > 1e-4f ? amax : 1e-4f) / 448.0f;
            if (ue8m0) scale = exp2f(ceilf(log2f(scale)));
            for (int64_t i = 0; i < quant_block; ++i) {
                uint16_t h = k[t * k_stride + g * quant_block + i];
                float x = is_fp16 ? fp16_bits_to_f32(h) : bf16_bits_to_f32(h);
                base[in_block * head_dim + g * quant_block + i] = f32_to_e4m3_bits(x / scale);
            }
            memcpy(base + block_size * head_dim + (in_block * nqb + g) * 4, &scale, 4);
        }
    }
    return 0;
}

/*
 * Gather of the sparse-indexer keys from their paged cache into token order, the torch statement
 * tests/test_cp_gather_indexer_k_quant_cache.py:85-116 of src/flaggems_vllm/ops/cp_gather_indexer_k_quant_cache.py:24-190:
 * request by request, token by token; rows of the outputs outside every request are not written.
 */
int dsv4_oracle_cp_gather_indexer(const uint8_t* cache, int64_t block_stride, uint8_t* k_out, int64_t k_out_stride, uint8_t* scale_out,
                                  int64_t scale_out_stride, const int32_t* block_table, int64_t block_table_stride,
                                  const int32_t* cu_seqlen, int64_t batch, int64_t num_tokens, int64_t block_size, int64_t head_dim,
                                  int64_t num_quant_blocks) {
    if (batch < 0 || block_size <= 0 || head_dim <= 0 || num_quant_blocks <= 0) return -1;
    for (int64_t b = 0; b < batch; ++b) {
        for (int64_t t = cu_seqlen[b]; t < cu_seqlen[b + 1]; ++t) {
            if (t < 0 || t >= num_tokens) return -2;
            int64_t off = t - cu_seqlen[b];
            const uint8_t* base = cache + (int64_t)block_table[b * block_table_stride + off / block_size] * block_stride;
            int64_t in_block = off % block_size;
            memcpy(k_out + t * k_out_stride, base + in_block * head_dim, (size_t)head_dim);
            memcpy(scale_out + t * scale_out_stride, base + block_size * head_dim + in_block * num_quant_blocks * 4,
                   (size_t)(num_quant_blocks * 4));
        }
    }
    return 0;
}

/*
 * Top-k positions inside a request -> cache slots, the expected-value loop of
 * tests/test_deepseek_v4_attention_compute_global_topk_indices_and_lens.py:92-108
 * (operator: src/flaggems_vllm/ops/deepseek_v4_attention_compute_global_topk_indices_and_lens.py:49-161).
 * is_valid may be NULL (every token valid).  Strides in elements.
 */
int dsv4_oracle_global_topk(const int32_t* local, int64_t local_stride, const int32_t* token_to_req, const int32_t* block_table,
                            int64_t block_table_stride, const int32_t* is_valid, int32_t* global, int64_t global_stride, int32_t* lens,
                            int64_t num_tokens, int64_t topk, int64_t block_size) {
    if (num_tokens < 0 || topk < 0 || block_size <= 0) return -1;
    for (int64_t t = 0; t < num_tokens; ++t) {
        int64_t req = token_to_req[t];
        int32_t count = 0;
        for (int64_t i = 0; i < topk; ++i) {
            int64_t pos = local[t * local_stride + i];
            if (pos >= 0) {
                global[t * global_stride + i] = (int32_t)(block_table[req * block_table_stride + pos / block_size] * block_size + pos % block_size);
                ++count;
            } else {
                global[t * global_stride + i] = -1;
            }
        }
        lens[t] = (!is_valid || is_valid[t]) ? count : 0;
    }
    return 0;
}

/*
 * Combined top-k / sliding-window index rows, the expected-value loop of
 * tests/test_deepseek_v4_attention_combine_topk_swa_indices.py:129-152
 * (operator: src/flaggems_vllm/ops/deepseek_v4_attention_combine_topk_swa_indices.py:30-161).
 * Rows of tokens that no request covers are not written.  Positions are taken as non-negative.
 */
int dsv4_oracle_combine_topk_swa(const int32_t* topk_indices, int64_t topk_stride, int64_t topk_width, const int32_t* query_start_loc,
                                 const int32_t* seq_lens, const int32_t* gather_lens, int32_t* combined, int64_t combined_stride,
                                 int64_t combined_width, int32_t* lens, int64_t num_reqs, int64_t num_tokens, int64_t window,
                                 int64_t compress_ratio, int64_t topk, int64_t m, int64_t n) {
    if (num_reqs < 0 || compress_ratio <= 0 || topk > topk_width || topk + window > combined_width) return -1;
    for (int64_t b = 0; b < num_reqs; ++b) {
        int64_t start = query_start_loc[b] - query_start_loc[0], end = query_start_loc[b + 1] - query_start_loc[0];
        int64_t start_pos = seq_lens[b] - (end - start), gather_start = seq_lens[b] - gather_lens[b];
        for (int64_t t = start; t < end; ++t) {
            if (t < 0 || t >= num_tokens) return -2;
            int64_t pos = start_pos + (t - start);
            if (pos < 0) return -3;
            int64_t topk_len = (pos + 1) / compress_ratio < topk ? (pos + 1) / compress_ratio : topk;
            int64_t swa_len = pos + 1 < window ? pos + 1 : window;
            int32_t* row = combined + t * combined_stride;
            for (int64_t c = 0; c < combined_width; ++c) row[c] = -1;
            for (int64_t i = 0; i < topk_len; ++i) row[i] = (int32_t)(topk_indices[t * topk_stride + i] + m * b);
            for (int64_t j = 0; j < swa_len; ++j) row[topk_len + j] = (int32_t)(m * b + n + j + pos - swa_len + 1 - gather_start);
            lens[t] = (int32_t)(topk_len + swa_len);
        }
    }
    return 0;
}

/*
 * Top-k positions per row, the torch statements tests/test_top_k_per_row_decode.py:111-124 and
 * tests/test_top_k_per_row_prefill.py:80-99 (torch.topk on the valid range of each row): the k = min(top_k, len)
 * largest values by a full sort (ties: lower position first), positions relative to the range start, then -1.
 * The upstream tests compare the selected VALUES as multisets, not the positions.
 */
typedef struct { float v; int32_t i; } oracle_pair;
static int oracle_pair_desc(const void* a, const void* b) {
    const oracle_pair *x = (const oracle_pair*)a, *y = (const oracle_pair*)b;
    if (x->v > y->v) return -1;
    if (x->v < y->v) return 1;
    return x->i < y->i ? -1 : (x->i > y->i ? 1 : 0);
}
int dsv4_oracle_top_k_per_row(const float* logits, int64_t stride0, int64_t stride1, const int32_t* starts, const int32_t* ends,
                              int32_t* indices, int64_t num_rows, int64_t vocab, int64_t top_k) {
    if (num_rows < 0 || vocab < 0 || top_k < 0) return -1;
    oracle_pair* buf = (oracle_pair*)malloc((size_t)(vocab > 0 ? vocab : 1) * sizeof(oracle_pair));
    if (!buf) return -2;
    for (int64_t r = 0; r < num_rows; ++r) {
        int64_t s = starts[r] < 0 ? 0 : starts[r], e = ends[r] > vocab ? vocab : ends[r];
        int64_t len = e > s ? e - s : 0, k = len < top_k ? len : top_k;
        for (int64_t i = 0; i < len; ++i) buf[i].v = logits[r * stride0 + (s + i) * stride1], buf[i].i = (int32_t)i;
        qsort(buf, (size_t)len, sizeof(oracle_pair), oracle_pair_desc);
        for (int64_t j = 0; j < top_k; ++j) indices[r * top_k + j] = j < k ? buf[j].i : -1;
    }
    free(buf);
    return 0;
}

/*
 * Per-token-group FP8 quantisation, the torch statement tests/test_per_token_group_quant_fp8.py:53-89 of
 * src/flaggems_vllm/ops/per_token_group_quant_fp8.py:25-330: scale = max(amax, eps) * (1/448) in fp32, made
 * exp2(ceil(log2(max(scale, 1e-10)))) when ue8m0; bytes = e4m3(clamp(x / scale, -448, 448)).  The statement clamps the
 * maximum while it still has the input's type (:68), so eps takes effect rounded to bf16 (1e-10 -> 1.0004e-10).
 * act_quant_rules: the statement of `act_quant` instead (tests/test_act_quant.py:49-99 of src/flaggems_vllm/ops/act_quant.py):
 * eps applied in fp32 and bytes = e4m3(clamp(x * (1/scale))).
 * x bf16 [rows, cols] with a row stride in elements; out contiguous; scale of (row, group) at
 * row*scale_stride_row + group*scale_stride_group.
 */
int dsv4_oracle_group_quant_fp8(const uint16_t* x, int64_t x_stride, uint8_t* out, float* scales, int64_t scale_stride_row,
                                int64_t scale_stride_group, int64_t rows, int64_t cols, int64_t group_size, float eps, int ue8m0,
                                int act_quant_rules) {
    if (rows < 0 || cols < 0 || group_size <= 0 || cols % group_size != 0) return -1;
    const float inv_max = 1.0f / 448.0f;
    if (!act_quant_rules) eps = bf16_bits_to_f32(f32_to_bf16_bits(eps));
    for (int64_t r = 0; r < rows; ++r) {
        for (int64_t g = 0; g < cols / group_size; ++g) {
            const uint16_t* src = x + r * x_stride + g * group_size;
            float amax = 0.0f;
            for (int64_t i = 0; i < group_size; ++i) {
                float a = fabsf(bf16_bits_to_f32(src[i]));
                if (a > amax) amax = a;
            }
            float scale = (amax > eps ? amax : eps) * inv_max;
            if (ue8m0) scale = exp2f(ceilf(log2f(scale > 1e-10f ? scale : 1e-10f)));
            for (int64_t i = 0; i < group_size; ++i) {
                float q = act_quant_rules ? bf16_bits_to_f32(src[i]) * (1.0f / scale) : bf16_bits_to_f32(src[i]) / scale;
                q = q > 448.0f ? 448.0f : (q < -448.0f ? -448.0f : q);
                out[r * cols + g * group_size + i] = f32_to_e4m3_bits(q);
            }
            scales[r * scale_stride_row + g * scale_stride_group] = scale;
        }
    }
    return 0;
}

/* e2m1 code of |v| <= 6 with the tie rule of tests/test_fused_indexer_q_rope_quant.py:81-92 (nearest, ties to even). */
static inline uint8_t e2m1_code(float v) {
    float a = fabsf(v);
    uint8_t code = 0;
    if (a > 0.25f) code = 1;
    if (a >= 0.75f) code = 2;
    if (a > 1.25f) code = 3;
    if (a >= 1.75f) code = 4;
    if (a > 2.5f) code = 5;
    if (a >= 3.5f) code = 6;
    if (a > 5.0f) code = 7;
    uint32_t u;
    memcpy(&u, &v, 4);
    return (uint8_t)(code | ((u >> 31) << 3));
}

/*
 * Sparse-indexer q prologue, the torch statement tests/test_fused_indexer_q_rope_quant.py:48-113 of
 * src/flaggems_vllm/ops/fused_indexer_q_rope_quant.py:69-280.  q bf16 [T, H, D] dense; cos_sin fp32 [max_pos, rot_dim];
 * weights fp32 [T, H] (already widened).  fp4 == 0: out e4m3 [T, H, D], weights_out = w*scale*softmax*head.
 * fp4 != 0: out [T, H, D/2] packed e2m1, scales [T, H, D/32] bytes, weights_out = w*softmax*head.
 */
int dsv4_oracle_indexer_q_rope_quant(const int64_t* positions, const uint16_t* q, const float* cos_sin, int64_t rot_dim,
                                     const float* weights, float softmax_scale, float head_scale, int64_t num_tokens,
                                     int64_t num_heads, int64_t head_dim, int fp4, uint8_t* out, uint8_t* scales,
                                     float* weights_out) {
    if (num_tokens < 0 || head_dim <= 0 || head_dim > 1024 || rot_dim > head_dim || rot_dim % 2) return -1;
    const int64_t nope = head_dim - rot_dim, half = rot_dim / 2;
    for (int64_t t = 0; t < num_tokens; ++t) {
        const float* cs = cos_sin + positions[t] * rot_dim;
        for (int64_t h = 0; h < num_heads; ++h) {
            const uint16_t* row = q + (t * num_heads + h) * head_dim;
            float x[1024];
            for (int64_t i = 0; i < nope; ++i) x[i] = bf16_bits_to_f32(row[i]);
            for (int64_t j = 0; j < half; ++j) {
                float e = bf16_bits_to_f32(row[nope + 2 * j]), o = bf16_bits_to_f32(row[nope + 2 * j + 1]);
                float ec = e * cs[j], os = o * cs[half + j], oc = o * cs[j], es = e * cs[half + j];
                x[nope + 2 * j] = bf16_bits_to_f32(f32_to_bf16_bits(ec - os));
                x[nope + 2 * j + 1] = bf16_bits_to_f32(f32_to_bf16_bits(oc + es));
            }
            float w = weights[t * num_heads + h];
            if (!fp4) {
                float amax = 0.0f;
                for (int64_t i = 0; i < head_dim; ++i) amax = fabsf(x[i]) > amax ? fabsf(x[i]) : amax;
                float scale = exp2f(ceilf(log2f((amax > 1e-4f ? amax : 1e-4f) / 448.0f)));
                for (int64_t i = 0; i < head_dim; ++i) out[(t * num_heads + h) * head_dim + i] = f32_to_e4m3_bits(x[i] / scale);
                w = w * scale;
            } else {
                for (int64_t b = 0; b < head_dim / 32; ++b) {
                    float amax = 0.0f;
                    for (int i = 0; i < 32; ++i) amax = fabsf(x[32 * b + i]) > amax ? fabsf(x[32 * b + i]) : amax;
                    const float floor_ = 6.0f * 1.17549435e-38f;
                    float lr = ceilf(log2f((amax > floor_ ? amax : floor_) / 6.0f));
                    lr = lr < -127.0f ? -127.0f : (lr > 127.0f ? 127.0f : lr);
                    float scale = exp2f(lr);
                    scales[(t * num_heads + h) * (head_dim / 32) + b] = (uint8_t)(lr + 127.0f);
                    for (int i = 0; i < 32; i += 2) {
                        float lo = x[32 * b + i] / scale, hi = x[32 * b + i + 1] / scale;
                        lo = lo < -6.0f ? -6.0f : (lo > 6.0f ? 6.0f : lo);
                        hi = hi < -6.0f ? -6.0f : (hi > 6.0f ? 6.0f : hi);
                        out[(t * num_heads + h) * (head_dim / 2) + (32 * b + i) / 2] = (uint8_t)(e2m1_code(lo) | (e2m1_code(hi) << 4));
                    }
                }
            }
            w = w * softmax_scale;
            weights_out[t * num_heads + h] = w * head_scale;
        }
    }
    return 0;
}

/*
 * Exhaustive check of the division shortcuts the CUDA quantisers use when their scales are not powers of two.
 * Once per group they form y within one ulp of RN(1/s) (approximate reciprocal + one Newton step) and
 * y_lo = RN(fma(-s, y, 1) * y); per value then either
 *   form 2 ("two-term"):   q = fma(x, y, RN(x * y_lo)), used for s <= 2^100 only (y_lo would be subnormal beyond), or
 *   form 3 ("corrected"):  q0 = RN(x * y), r = fma(-s, q0, x), q = fma(r, y, q0), used for any s.
 * For every non-negative finite bf16 amax, s = RN(max(amax, eps) * RN(1/448)), every bf16 x with 0 <= x <= amax, and
 * y = RN(1/s) moved by `y_ulps` (-1, 0 or +1: the three values the device's y can take), counts the pairs whose
 * e4m3 byte differs from that of the IEEE quotient RN(x/s) (`byte_mismatches`) and, for information, those whose fp32
 * value differs (`value_mismatches`; for form 2 these are quotients so far below the group maximum that their byte is
 * zero either way).  Pairs outside a form's range are not counted.  Negative x behave symmetrically.
 * Returns the number of pairs examined.
 */
__attribute__((target("fma"))) static inline float fma_hw(float a, float b, float c) { return __builtin_fmaf(a, b, c); }

int64_t dsv4_oracle_check_division_shortcut(float eps, int form, int y_ulps, int64_t* byte_mismatches, int64_t* value_mismatches) {
    int64_t pairs = 0, bytes = 0, values = 0;
    const float inv448 = (float)(1.0 / 448.0);
    const int have_fma = __builtin_cpu_supports("fma");
#pragma omp parallel for schedule(dynamic, 64) reduction(+ : pairs, bytes, values)
    for (int32_t ia = 0; ia < 0x7f80; ++ia) {
        float amax = bf16_bits_to_f32((uint16_t)ia);
        float s = (amax < eps ? eps : amax) * inv448;
        if (form == 2 && !(s <= 0x1p100f)) continue;
        float y = 1.0f / s;
        uint32_t y_bits;
        memcpy(&y_bits, &y, 4);
        y_bits += (uint32_t)y_ulps;
        memcpy(&y, &y_bits, 4);
        float residual = have_fma ? fma_hw(-s, y, 1.0f) : fmaf(-s, y, 1.0f);
        float y_lo = residual * y;
        for (int32_t ix = 0; ix <= ia; ++ix) {
            float x = bf16_bits_to_f32((uint16_t)ix);
            float want = x / s, q;
            if (form == 2) {
                float c = x * y_lo;
                q = have_fma ? fma_hw(x, y, c) : fmaf(x, y, c);
            } else {
                float q0 = x * y;
                float r = have_fma ? fma_hw(-s, q0, x) : fmaf(-s, q0, x);
                q = have_fma ? fma_hw(r, y, q0) : fmaf(r, y, q0);
            }
            pairs++;
            if (q != want) values++;
            float qc = q > 448.0f ? 448.0f : q, wc = want > 448.0f ? 448.0f : want;
            if (f32_to_e4m3_bits(qc) != f32_to_e4m3_bits(wc)) bytes++;
        }
    }
    *byte_mismatches = bytes;
    *value_mismatches = values;
    return pairs;
}

const char* dsv4_oracle_version(void) { return "dsv4-oracle 1"; }
