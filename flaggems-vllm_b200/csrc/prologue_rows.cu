// Variant ROWS of the fused prologue: one launch, one warp per 512-element row,
// 16-byte vector loads/stores through registers.
//
// Grid = [kv CTAs][q CTAs].  A q CTA owns a tile of TILE = WARPS*RPW consecutive
// rows of q viewed as [num_tokens*num_heads, 512]; it issues all of its row
// loads first, stages the cos|sin rows of the (usually one) tokens the tile
// touches in shared memory while those loads are in flight, reduces the sum of
// squares per warp with shuffles, synchronises once and writes the rows back in
// place.  A kv CTA handles WARPS tokens of the latent KV, one per warp; those
// CTAs come first in the grid so they never form the tail of the launch.
//
// Replaces the per-(token, head) Triton programs of the reference
// (src/flaggems_vllm/ops/fused_deepseek_v4_qnorm_rope_kv_rope_quant_insert.py:45-286).
#include "dsv4_common.cuh"

namespace dsv4 {
namespace {

template <int RPW, int WARPS, int MIN_CTAS, bool CHECKED>
__global__ void __launch_bounds__(WARPS * 32, MIN_CTAS) prologue_rows_kernel(const PrologueParams p, const int64_t kv_ctas) {
    constexpr int TILE = RPW * WARPS;
    constexpr int MAX_TOKENS = TILE + 1;  // a tile of TILE rows touches at most TILE tokens (+1 slack)
    __shared__ __align__(16) float cs_smem[MAX_TOKENS][kRopeDim];
    __shared__ int bad_token[MAX_TOKENS];

    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;

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
        const uint8_t* row = p.kv + t * kRowBytes;
        const uint4 a = ld_stream16(row + 16 * lane);
        const uint4 b = ld_stream16(row + 512 + 16 * lane);
        float4 c = make_float4(0.f, 0.f, 0.f, 0.f), s = c;
        if (lane >= kFirstRopeLane) {
            const float* cs = p.cos_sin + pos * kRopeDim + 4 * (lane - kFirstRopeLane);
            c = ld_readonly_f4(cs);
            s = ld_readonly_f4(cs + 32);
        }
        const int64_t block = slot / p.block_size, in_block = slot - block * p.block_size;
        uint8_t* base = p.k_cache + block * p.block_stride;
        kv_row_to_cache(a, b, lane, c, s, base + in_block * kTokenDataBytes,
                        base + p.block_size * kTokenDataBytes + in_block * kScaleBytes, p.cache_aligned16 != 0);
        return;
    }

    // ---- q rows: RMSNorm + RoPE tail, in place
    const int64_t total_rows = p.num_tokens * p.num_heads;
    const int64_t tile_row0 = (static_cast<int64_t>(blockIdx.x) - kv_ctas) * TILE;
    const int64_t row0 = tile_row0 + warp * RPW;

    uint4 a[RPW], b[RPW];
#pragma unroll
    for (int i = 0; i < RPW; ++i) {
        a[i] = b[i] = make_uint4(0u, 0u, 0u, 0u);
        if (row0 + i < total_rows) {
            const uint8_t* row = p.q + (row0 + i) * kRowBytes;
            a[i] = ld_stream16(row + 16 * lane);
            b[i] = ld_stream16(row + 512 + 16 * lane);
        }
    }

    // cos|sin rows of the tokens this tile touches -> shared memory (16 threads per token)
    const int64_t first_token = tile_row0 / p.num_heads;
    const int64_t last_row = (tile_row0 + TILE < total_rows ? tile_row0 + TILE : total_rows) - 1;
    const int n_tokens = static_cast<int>(last_row / p.num_heads - first_token) + 1;
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

    float r[RPW];
#pragma unroll
    for (int i = 0; i < RPW; ++i) r[i] = inv_rms(warp_sum(sumsq8(b[i], sumsq8(a[i], 0.0f))), p.eps);
    // Keep the rows packed across the barrier (16 registers per pair of rows instead of 32
    // unpacked floats): the empty asm makes the compiler unpack them again for the store.
#pragma unroll
    for (int i = 0; i < RPW; ++i) {
        asm volatile("" : "+r"(a[i].x), "+r"(a[i].y), "+r"(a[i].z), "+r"(a[i].w));
        asm volatile("" : "+r"(b[i].x), "+r"(b[i].y), "+r"(b[i].z), "+r"(b[i].w));
    }

    __syncthreads();

    const int my_token0 = static_cast<int>(row0 / p.num_heads - first_token);
    const int rem0 = static_cast<int>(row0 - (first_token + my_token0) * p.num_heads);
#pragma unroll
    for (int i = 0; i < RPW; ++i) {
        if (row0 + i >= total_rows) break;
        const int64_t within = static_cast<int64_t>(rem0) + i;
        const int tok = my_token0 + static_cast<int>(within / p.num_heads);
        if (CHECKED && bad_token[tok]) continue;
        uint8_t* row = p.q + (row0 + i) * kRowBytes;
        st_stream16(row + 16 * lane, scale8(a[i], r[i]));
        uint4 out_b;
        if (lane >= kFirstRopeLane) {
            const float4 c = *reinterpret_cast<const float4*>(&cs_smem[tok][4 * (lane - kFirstRopeLane)]);
            const float4 s = *reinterpret_cast<const float4*>(&cs_smem[tok][32 + 4 * (lane - kFirstRopeLane)]);
            out_b = scale_rotate8(b[i], r[i], c, s);
        } else {
            out_b = scale8(b[i], r[i]);
        }
        st_stream16(row + 512 + 16 * lane, out_b);
    }
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
    if (checked)
        prologue_rows_kernel<RPW, WARPS, MIN_CTAS, true><<<static_cast<unsigned>(grid), WARPS * 32, 0, stream>>>(p, kv_ctas);
    else
        prologue_rows_kernel<RPW, WARPS, MIN_CTAS, false><<<static_cast<unsigned>(grid), WARPS * 32, 0, stream>>>(p, kv_ctas);
    count_launch();
    return cudaGetLastError();
}

}  // namespace

cudaError_t launch_prologue_rows(const PrologueParams& p, bool checked, cudaStream_t stream) {
#ifdef DSV4_ROWS_RPW
    return launch<DSV4_ROWS_RPW, DSV4_ROWS_WARPS, DSV4_ROWS_MIN_CTAS>(p, checked, stream);
#else
    return launch<2, 8, 5>(p, checked, stream);
#endif
}

}  // namespace dsv4
