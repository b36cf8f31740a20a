// Variant ROWS of the fused prologue: one launch, one warp per 512-element row,
// 16-byte vector loads/stores through registers.
//
// Grid = [kv CTAs][q CTAs].  A q CTA owns a tile of TILE = WARPS*RPW consecutive
// rows of q viewed as [num_tokens*num_heads, 512]; it issues all of its row
// loads first, stages the cos|sin rows of the (usually one) tokens the tile
// touches in shared memory while those loads are in flight, synchronises once,
// then each warp finishes its rows one after the other: sum of squares reduced
// with shuffles, scale, rotate, store in place.  A kv CTA handles WARPS tokens of the latent KV, one per warp; those
// CTAs come first in the grid so they never form the tail of the launch.
//
// Replaces the per-(token, head) Triton programs of the reference
// (src/flaggems_vllm/ops/fused_deepseek_v4_qnorm_rope_kv_rope_quant_insert.py:45-286).
#include "dsv4_common.cuh"

namespace dsv4 {
namespace {

// PADDED: out-of-place form (vLLM >= 0.22 calls the operator that way): rows go to p.q_out with out_heads heads per
// token and the CTAs after the q tiles zero-fill the extra heads.
// Programmatic dependent launch (sm_90+): the kernel may start while the preceding kernel of the stream still runs;
// `wait` returns once that kernel has completed and its writes are visible (a no-op for an ordinary launch), and
// `launch_dependents` lets the next kernel of the stream start its own independent part.
__device__ __forceinline__ void wait_for_preceding_kernel() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void let_next_kernel_start() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// STAGED: the cos|sin rows of the tile's tokens go through shared memory (one fetch per CTA, one barrier).  Without
// it every warp fetches position and table row of its own rows straight into registers (lane i holds cosine i and
// sine i): 256 more bytes from L2 per row, but no barrier and no shared-memory round trip in the dependent chain
// position -> table row, which is what a launch of a few waves waits for.
template <int RPW, int WARPS, int MIN_CTAS, bool CHECKED, bool PADDED, int PDL = 0, bool STAGED = true>
__global__ void __launch_bounds__(WARPS * 32, MIN_CTAS) prologue_rows_kernel(const PrologueParams p, const int64_t kv_ctas) {
    static_assert(STAGED || !CHECKED, "the range-checked build marks bad tokens in shared memory");
    constexpr int TILE = RPW * WARPS;
    constexpr int MAX_TOKENS = TILE + 1;  // a tile of TILE rows touches at most TILE tokens (+1 slack)
    __shared__ __align__(16) float cs_smem[MAX_TOKENS][kRopeDim];
    __shared__ int bad_token[MAX_TOKENS];

    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;

    // PDL 2: programmatic dependent launch with ordinary stream semantics - nothing is read before the preceding kernel
    // of the stream has finished; what overlaps with that kernel's tail is only this kernel's own launch.
    // PDL 1: positions, slots and table rows are read first and only q, kv and the cache wait (the caller promises
    // that the preceding kernel does not write the former).
    if (PDL == 2) wait_for_preceding_kernel();
    if (static_cast<int64_t>(blockIdx.x) < kv_ctas) {
        // ---- latent KV: RoPE tail + UE8M0/e4m3 quantisation + scatter through slot_mapping
        const int64_t t = static_cast<int64_t>(blockIdx.x) * WARPS + warp;
        if (t >= p.num_tokens_insert) return;
        const int64_t slot = p.slot_mapping[t];
        if (slot < 0) return;
        const int64_t pos = p.position_ids[t];
        if (CHECKED) {
            const bool bad_pos = pos < 0 || pos >= p.max_pos, bad_slot = slot >= p.num_slots;
            if (bad_pos || bad_slot) {
                if (lane == 0) atomicOr(p.status, (bad_pos ? 1 : 0) | (bad_slot ? 2 : 0));
                return;
            }
        }
        float4 c = make_float4(0.f, 0.f, 0.f, 0.f), s = c;
        if (lane >= kFirstRopeLane) {
            const float* cs = p.cos_sin + pos * kRopeDim + 4 * (lane - kFirstRopeLane);
            c = ld_readonly_f4(cs);
            s = ld_readonly_f4(cs + 32);
        }
        if (PDL == 1) wait_for_preceding_kernel();  // kv (and the cache) may still be written by it
        const uint8_t* row = p.kv + t * kRowBytes;
        const uint4 a = ld_stream16(row + 16 * lane);
        const uint4 b = ld_stream16(row + 512 + 16 * lane);
        if (PDL) let_next_kernel_start();
        const int64_t block = slot / p.block_size, in_block = slot - block * p.block_size;
        uint8_t* base = p.k_cache + block * p.block_stride;
        kv_row_to_cache(a, b, lane, c, s, base + in_block * kTokenDataBytes,
                        base + p.block_size * kTokenDataBytes + in_block * kScaleBytes, p.cache_aligned16 != 0);
        return;
    }

    // ---- q rows: RMSNorm + RoPE tail, in place (row and token indices fit 32 bits: host-checked)
    const uint32_t total_rows = static_cast<uint32_t>(p.num_tokens * p.num_heads);
    const uint32_t tile_row0 = (blockIdx.x - static_cast<uint32_t>(kv_ctas)) * TILE;
    const uint32_t row0 = tile_row0 + warp * RPW;
    if (PADDED && tile_row0 >= total_rows) {
        // zero-fill: padding row j is head num_heads + j % extra of token j / extra
        const uint32_t extra = static_cast<uint32_t>(p.out_heads - p.num_heads);
        const uint32_t pad_rows = static_cast<uint32_t>(p.num_tokens) * extra;
        const uint32_t first_pad_tile = (total_rows + TILE - 1) / TILE * TILE;
#pragma unroll
        for (int i = 0; i < RPW; ++i) {
            const uint32_t j = row0 - first_pad_tile + i;
            if (j >= pad_rows) break;
            const uint32_t tok = j / extra;
            uint8_t* dst = p.q_out + (static_cast<uint64_t>(tok) * p.out_heads + p.num_heads + (j - tok * extra)) * kRowBytes;
            const uint4 z = make_uint4(0u, 0u, 0u, 0u);
            st_stream16(dst + 16 * lane, z);
            st_stream16(dst + 512 + 16 * lane, z);
        }
        return;
    }

    // 1. the row loads of the CTA (A/B/T layout, 16 + 16 + 4 bytes per lane)
    uint4 a[RPW], b[RPW];
    uint32_t tail[RPW];
    const auto issue_row_loads = [&]() {
#pragma unroll
        for (int i = 0; i < RPW; ++i) {
            a[i] = b[i] = make_uint4(0u, 0u, 0u, 0u);
            tail[i] = 0u;
            if (row0 + i < total_rows) {
                const uint8_t* row = p.q + static_cast<uint64_t>(row0 + i) * kRowBytes;
                a[i] = ld_inplace16(row + 16 * lane);
                if (lane < kFirstRopeLane) b[i] = ld_inplace16(row + 512 + 16 * lane);
                tail[i] = ld_inplace4(row + 2 * kNopeDim + 4 * lane);
            }
        }
    };
    // 2. cos|sin rows of the tokens this tile touches -> shared memory (16 threads per token, 16 bytes each)
    const uint32_t first_token = fast_div(tile_row0, p.heads_mul, p.heads_shift);
    const uint32_t last_row = (tile_row0 + TILE < total_rows ? tile_row0 + TILE : total_rows) - 1;
    const int n_tokens = static_cast<int>(fast_div(last_row, p.heads_mul, p.heads_shift) - first_token) + 1;
    const auto stage_cos_sin = [&]() {
        for (int j = threadIdx.x >> 4; j < n_tokens; j += WARPS * 2) {
            const int part = threadIdx.x & 15;
            int64_t pos = p.position_ids[first_token + j];
            if (CHECKED) {
                const bool bad = pos < 0 || pos >= p.max_pos;
                if (part == 0) {
                    bad_token[j] = bad ? 1 : 0;
                    if (bad) atomicOr(p.status, 1);
                }
                if (bad) pos = 0;
            }
            *reinterpret_cast<float4*>(&cs_smem[j][4 * part]) = ld_readonly_f4(p.cos_sin + pos * kRopeDim + 4 * part);
        }
    };
    // without staging: cosine and sine of this lane's pair for each row of the warp, straight from the table
    float cos_r[RPW], sin_r[RPW];
    const auto fetch_cos_sin = [&]() {
#pragma unroll
        for (int i = 0; i < RPW; ++i) {
            cos_r[i] = sin_r[i] = 0.f;
            if (row0 + i < total_rows) {
                const int64_t pos = p.position_ids[fast_div(row0 + i, p.heads_mul, p.heads_shift)];
                const float* cs = p.cos_sin + pos * kRopeDim + lane;
                cos_r[i] = __ldg(cs), sin_r[i] = __ldg(cs + 32);
            }
        }
    };
    if (PDL == 1) {
        // the table rows first (they do not depend on the preceding kernel), q only once that kernel has finished
        if (STAGED) stage_cos_sin(); else fetch_cos_sin();
        wait_for_preceding_kernel();
        issue_row_loads();
        let_next_kernel_start();
    } else {
        // every row load goes out first; the table rows are fetched while they fly
        issue_row_loads();
        if (STAGED) stage_cos_sin(); else fetch_cos_sin();
        if (PDL) let_next_kernel_start();
    }
    if (STAGED) __syncthreads();

    // 3. one row at a time: unpack once, reduce, scale, rotate the lane's pair, store
#pragma unroll
    for (int i = 0; i < RPW; ++i) {
        if (row0 + i >= total_rows) break;
        const uint32_t token = fast_div(row0 + i, p.heads_mul, p.heads_shift);
        const int tok = static_cast<int>(token - first_token);
        if (CHECKED && bad_token[tok]) continue;
        float xa[8], xb[8];
        unpack8(a[i], xa), unpack8(b[i], xb);
        const float r = row_inv_rms(xa, xb, tail[i], p.eps);
        scale8(xa, r), scale8(xb, r);
        uint8_t* row = PADDED ? p.q_out + (static_cast<uint64_t>(row0 + i) + static_cast<uint64_t>(token) * (p.out_heads - p.num_heads)) * kRowBytes
                              : p.q + static_cast<uint64_t>(row0 + i) * kRowBytes;
        st_stream16(row + 16 * lane, pack8(xa));
        if (lane < kFirstRopeLane) st_stream16(row + 512 + 16 * lane, pack8(xb));
        st_stream4(row + 2 * kNopeDim + 4 * lane,
                   scale_rotate_pair(tail[i], r, STAGED ? cs_smem[tok][lane] : cos_r[i], STAGED ? cs_smem[tok][32 + lane] : sin_r[i]));
    }
}

// Any 2-byte alignment of q and kv (a contiguous view that starts a few elements into its storage) and any 4-byte
// alignment of the table: the reference only asks for contiguous tensors.  One warp per row in a "pair" layout - lane l
// holds the (even, odd) pairs l, l + 32, ..., l + 224 of the row, read and written with 2-byte accesses - so pair l + 224 is
// the lane's rotary pair and the pairs l + 32g are one quantisation group g of a latent-KV row.  Same arithmetic as the
// kernels above (the sum of squares is grouped differently, within the freedom the mean has anyway); cache bytes are
// identical.  Only this plain form exists for such pointers: no range-checked and no out-of-place variant.
template <int WARPS>
__global__ void __launch_bounds__(WARPS * 32) prologue_rows_any_alignment_kernel(const PrologueParams p, const int64_t kv_ctas) {
    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
    const bool is_kv = static_cast<int64_t>(blockIdx.x) < kv_ctas;
    const int64_t r = (is_kv ? static_cast<int64_t>(blockIdx.x) : static_cast<int64_t>(blockIdx.x) - kv_ctas) * WARPS + warp;
    int64_t token = r, slot = 0;
    if (is_kv) {
        if (r >= p.num_tokens_insert) return;
        slot = p.slot_mapping[r];
        if (slot < 0) return;
    } else {
        if (r >= p.num_tokens * p.num_heads) return;
        token = r / p.num_heads;
    }
    const float* cs = p.cos_sin + p.position_ids[token] * kRopeDim;
    const float c = cs[lane], sn = cs[32 + lane];
    const uint16_t* in = reinterpret_cast<const uint16_t*>(is_kv ? p.kv : p.q) + r * (kRowBytes / 2);
    float e[8], o[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) e[j] = bf16_lo(in[2 * (lane + 32 * j)]), o[j] = bf16_lo(in[2 * (lane + 32 * j) + 1]);
    if (!is_kv) {
        sumsq_t acc = sumsq_t(0);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
#if DSV4_EXACT_SUMSQ
            acc = fma(static_cast<double>(o[j]), static_cast<double>(o[j]), fma(static_cast<double>(e[j]), static_cast<double>(e[j]), acc));
#else
            acc = fmaf(o[j], o[j], fmaf(e[j], e[j], acc));
#endif
        }
        const float rr = inv_rms(warp_sum(acc), p.eps);
        uint16_t* out = reinterpret_cast<uint16_t*>(p.q) + r * (kRowBytes / 2);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const uint32_t packed = static_cast<uint32_t>(in[2 * (lane + 32 * j)]) | (static_cast<uint32_t>(in[2 * (lane + 32 * j) + 1]) << 16);
            const uint32_t y = j == 7 ? scale_rotate_pair(packed, rr, c, sn) : pack_bf16x2(__fmul_rn(e[j], rr), __fmul_rn(o[j], rr));
            out[2 * (lane + 32 * j)] = static_cast<uint16_t>(y & 0xffffu);
            out[2 * (lane + 32 * j) + 1] = static_cast<uint16_t>(y >> 16);
        }
        return;
    }
    const int64_t block = slot / p.block_size, in_block = slot - block * p.block_size;
    uint8_t* base = p.k_cache + block * p.block_stride;
    uint8_t* data = base + in_block * kTokenDataBytes;
    uint8_t* scales = base + p.block_size * kTokenDataBytes + in_block * kScaleBytes;
#pragma unroll
    for (int g = 0; g < 7; ++g) {
        float amax = fmaxf(fabsf(e[g]), fabsf(o[g]));
#pragma unroll
        for (int m = 16; m > 0; m >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, m));
        const uint32_t code = ue8m0_code(amax);
        const float scale = __uint_as_float(code << 23);
        const uint32_t bytes = pack_e4m3x4(__fdiv_rn(e[g], scale), __fdiv_rn(o[g], scale), 0.f, 0.f);
        data[64 * g + 2 * lane] = static_cast<uint8_t>(bytes & 0xffu);
        data[64 * g + 2 * lane + 1] = static_cast<uint8_t>((bytes >> 8) & 0xffu);
        if (lane == 0) scales[g] = static_cast<uint8_t>(code);
    }
    if (lane == 0) scales[7] = 0;
    const uint32_t rot = pack_bf16x2(__fsub_rn(__fmul_rn(e[7], c), __fmul_rn(o[7], sn)), __fadd_rn(__fmul_rn(e[7], sn), __fmul_rn(o[7], c)));
#pragma unroll
    for (int b = 0; b < 4; ++b) data[kNopeDim + 4 * lane + b] = static_cast<uint8_t>((rot >> (8 * b)) & 0xffu);
}

template <int RPW, int WARPS, int MIN_CTAS>
cudaError_t launch(const PrologueParams& p, bool checked, cudaStream_t stream) {
    constexpr int TILE = RPW * WARPS;
    const int64_t kv_ctas = (p.num_tokens_insert + WARPS - 1) / WARPS;
    const int64_t total_rows = p.num_tokens * p.num_heads;
    const int64_t q_ctas = (total_rows + TILE - 1) / TILE;
    const int64_t grid = kv_ctas + q_ctas;
    if (grid == 0) return cudaSuccess;
    if (grid > 0x7fffffffLL) return cudaErrorInvalidConfiguration;
    if (checked) {
        prologue_rows_kernel<RPW, WARPS, MIN_CTAS, true, false><<<static_cast<unsigned>(grid), WARPS * 32, 0, stream>>>(p, kv_ctas);
    } else if (p.pdl) {
        const auto kernel = p.pdl == 2 ? (p.table_staging ? prologue_rows_kernel<RPW, WARPS, MIN_CTAS, false, false, 2, true>
                                                          : prologue_rows_kernel<RPW, WARPS, MIN_CTAS, false, false, 2, false>)
                                       : (p.table_staging ? prologue_rows_kernel<RPW, WARPS, MIN_CTAS, false, false, 1, true>
                                                          : prologue_rows_kernel<RPW, WARPS, MIN_CTAS, false, false, 1, false>);
        cudaLaunchConfig_t config = {};
        config.gridDim = dim3(static_cast<unsigned>(grid)), config.blockDim = dim3(WARPS * 32), config.stream = stream;
        cudaLaunchAttribute attribute[1];
        attribute[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attribute[0].val.programmaticStreamSerializationAllowed = 1;
        config.attrs = attribute, config.numAttrs = 1;
        const cudaError_t err = cudaLaunchKernelEx(&config, kernel, p, kv_ctas);
        if (err != cudaSuccess) return err;
    } else if (p.table_staging) {
        prologue_rows_kernel<RPW, WARPS, MIN_CTAS, false, false><<<static_cast<unsigned>(grid), WARPS * 32, 0, stream>>>(p, kv_ctas);
    } else {
        prologue_rows_kernel<RPW, WARPS, MIN_CTAS, false, false, 0, false><<<static_cast<unsigned>(grid), WARPS * 32, 0, stream>>>(p, kv_ctas);
    }
    count_launch();
    return cudaGetLastError();
}

template <int RPW, int WARPS, int MIN_CTAS>
cudaError_t launch_padded(const PrologueParams& p, cudaStream_t stream) {
    constexpr int TILE = RPW * WARPS;
    const int64_t kv_ctas = (p.num_tokens_insert + WARPS - 1) / WARPS;
    const int64_t q_ctas = (p.num_tokens * p.num_heads + TILE - 1) / TILE;
    const int64_t pad_ctas = (p.num_tokens * (p.out_heads - p.num_heads) + TILE - 1) / TILE;
    const int64_t grid = kv_ctas + q_ctas + pad_ctas;
    if (grid == 0) return cudaSuccess;
    if (grid > 0x7fffffffLL) return cudaErrorInvalidConfiguration;
    prologue_rows_kernel<RPW, WARPS, MIN_CTAS, false, true><<<static_cast<unsigned>(grid), WARPS * 32, 0, stream>>>(p, kv_ctas);
    count_launch();
    return cudaGetLastError();
}

}  // namespace

cudaError_t launch_prologue_rows_any_alignment(const PrologueParams& p, cudaStream_t stream) {
    constexpr int WARPS = 4;
    const int64_t kv_ctas = (p.num_tokens_insert + WARPS - 1) / WARPS;
    const int64_t grid = kv_ctas + (p.num_tokens * p.num_heads + WARPS - 1) / WARPS;
    if (grid == 0) return cudaSuccess;
    if (grid > 0x7fffffffLL) return cudaErrorInvalidConfiguration;
    prologue_rows_any_alignment_kernel<WARPS><<<static_cast<unsigned>(grid), WARPS * 32, 0, stream>>>(p, kv_ctas);
    count_launch();
    return cudaGetLastError();
}

cudaError_t launch_prologue_rows(const PrologueParams& p, bool checked, cudaStream_t stream) {
#ifdef DSV4_ROWS_RPW
    return launch<DSV4_ROWS_RPW, DSV4_ROWS_WARPS, DSV4_ROWS_MIN_CTAS>(p, checked, stream);
#else
    // 2 rows per warp, 4 warps, 10 CTAs per SM (48 registers): the fastest of the swept shapes on B200
    return launch<2, 4, 10>(p, checked, stream);
#endif
}

cudaError_t launch_prologue_rows_padded(const PrologueParams& p, cudaStream_t stream) { return launch_padded<2, 4, 10>(p, stream); }

}  // namespace dsv4
