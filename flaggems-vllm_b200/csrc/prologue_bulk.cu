// Variant BULK of the fused prologue: persistent CTAs that move q through a ring of
// shared-memory stages with bulk asynchronous copies (the TMA engine, 1-D form), so that many
// KiB per SM are in flight without holding them in registers.
//
// Work is cut into tiles of TILE consecutive 1-KiB rows: first the latent-KV rows
// (kv viewed as [num_tokens_insert, 512]), then the q rows (q viewed as
// [num_tokens*num_heads, 512]); a tile is one contiguous byte range.  CTA c takes tiles
// c, c+gridDim, c+2*gridDim, ...  Roles inside a CTA (no role waits on another CTA):
//   warp 0  "loader"  : per tile, one bulk copy global->shared of the rows plus one 256-byte
//                        bulk copy per token of the tile for its cos|sin row, all completing on
//                        the stage's `full` mbarrier; positions are fetched two tiles ahead.
//   warp 1  "storer"  : when the workers are done with a stage, one bulk copy shared->global
//                        writes the rows back in place; once that copy has finished reading
//                        shared memory the stage is handed back to the loader (`empty`).
//   warps 2.. "workers": one warp per row: RMSNorm (shuffle reduction) + RoPE in shared memory
//                        for q tiles; RoPE + UE8M0/e4m3 quantisation + scatter to the paged
//                        cache with ordinary stores for KV tiles.
// Every mbarrier wait is bounded (PrologueParams::wait_cycles SM cycles, set per launch by the host); a wait that runs
// out sets bit 0 of the device-side error word (read with dsv4_device_error) and makes the CTA's roles leave their
// loops: the loader then waits, again bounded, for the copies it has already issued before the CTA ends.
//
// Replaces the per-(token, head) Triton programs of the reference
// (src/flaggems_vllm/ops/fused_deepseek_v4_qnorm_rope_kv_rope_quant_insert.py:45-286).
#include <mutex>

#include "dsv4_common.cuh"

namespace dsv4 {

__device__ int g_device_error = 0;

namespace {

constexpr int kKindQ = 0, kKindKV = 1, kKindDone = 2;
constexpr uint32_t kWaitLimit = 1u << 24;  // polls before a wait gives up, or PrologueParams::wait_cycles SM cycles, whichever comes first

struct __align__(16) TileHeader {
    uint32_t row0;         // first row of the tile in its tensor (rows and tokens fit 32 bits: host-checked)
    uint32_t first_token;  // token of row0
    uint32_t rem;          // row0 - first_token * num_heads (q tiles)
    int32_t nrows;
    int32_t ntok;
    int32_t kind;
    int32_t pad[2];
};

// ---- PTX wrappers -----------------------------------------------------------

__device__ __forceinline__ uint32_t smem_addr(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_addr(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_addr(bar)) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_addr(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done)
        : "r"(smem_addr(bar)), "r"(parity)
        : "memory");
    return done != 0;
}
// Bounded wait.  Returns false (and raises the abort flag) when the limit is reached or another
// role of the CTA has already given up.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag, long long limit_cycles) {
    if (mbar_try_wait(bar, parity)) return true;
    const long long start = clock64();
    for (uint32_t i = 0; i < kWaitLimit; ++i) {
        if (mbar_try_wait(bar, parity)) return true;
        if (*abort_flag) return false;
        if (clock64() - start > limit_cycles) break;
    }
    *abort_flag = 1;
    atomicOr(&g_device_error, 1);
    return false;
}
__device__ __forceinline__ void bulk_load(void* smem_dst, const void* gmem_src, uint32_t bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                     smem_addr(smem_dst)),
                 "l"(gmem_src), "r"(bytes), "r"(smem_addr(bar))
                 : "memory");
}
__device__ __forceinline__ void bulk_store(void* gmem_dst, const void* smem_src, uint32_t bytes) {
    asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(gmem_dst), "r"(smem_addr(smem_src)),
                 "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void bulk_wait_read() {
    asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void bulk_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void fence_barrier_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }

// ---- the kernel ---------------------------------------------------------------

template <int TILE, int STAGES, int WORKERS>
struct BulkLayout {
    static constexpr int kDataBytes = TILE * kRowBytes;
    static constexpr int kCosSinBytes = TILE * kCosSinRowBytes;
    static constexpr int kStageBytes = kDataBytes + kCosSinBytes;
    static constexpr int kHeaderOffset = STAGES * kStageBytes;
    static constexpr int kBarrierOffset = kHeaderOffset + STAGES * static_cast<int>(sizeof(TileHeader));
    static constexpr int kAbortOffset = kBarrierOffset + 3 * STAGES * 8;
    static constexpr int kTotalBytes = kAbortOffset + 16;
    static constexpr int kThreads = (WORKERS + 2) * 32;
};

template <int TILE, int STAGES, int WORKERS, int PENDING, int CTAS_PER_SM>
__global__ void __launch_bounds__((WORKERS + 2) * 32, CTAS_PER_SM)
prologue_bulk_kernel(const PrologueParams p, const uint32_t kv_tiles, const uint32_t total_tiles) {
    using L = BulkLayout<TILE, STAGES, WORKERS>;
    static_assert(TILE <= 32, "one loader lane per token of a tile");
    static_assert(PENDING >= 1 && PENDING < STAGES, "stores in flight must leave stages for loads");
    extern __shared__ __align__(128) uint8_t smem[];
    TileHeader* headers = reinterpret_cast<TileHeader*>(smem + L::kHeaderOffset);
    uint64_t* full = reinterpret_cast<uint64_t*>(smem + L::kBarrierOffset);
    uint64_t* done = full + STAGES;
    uint64_t* empty = done + STAGES;
    volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + L::kAbortOffset);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&done[s], WORKERS);
            mbar_init(&empty[s], 1);
        }
        *abort_flag = 0;
        fence_barrier_init();
        fence_async_smem();
    }
    __syncthreads();

    const uint32_t total_rows = static_cast<uint32_t>(p.num_tokens * p.num_heads);

    if (warp == 0) {
        // ------------------------------------------------------------ loader
        auto describe = [&](uint32_t tile) {
            TileHeader h;
            h.row0 = 0, h.first_token = 0, h.rem = 0, h.nrows = 0, h.ntok = 0, h.kind = kKindDone;
            if (tile >= total_tiles) return h;
            if (tile < kv_tiles) {
                h.kind = kKindKV;
                h.row0 = tile * TILE;
                const uint32_t left = static_cast<uint32_t>(p.num_tokens_insert) - h.row0;
                h.nrows = static_cast<int32_t>(left < TILE ? left : TILE);
                h.first_token = h.row0;
                h.ntok = h.nrows;
            } else {
                h.kind = kKindQ;
                h.row0 = (tile - kv_tiles) * TILE;
                const uint32_t left = total_rows - h.row0;
                h.nrows = static_cast<int32_t>(left < TILE ? left : TILE);
                h.first_token = fast_div(h.row0, p.heads_mul, p.heads_shift);
                h.rem = h.row0 - h.first_token * static_cast<uint32_t>(p.num_heads);
                h.ntok = static_cast<int32_t>(fast_div(h.row0 + h.nrows - 1, p.heads_mul, p.heads_shift) - h.first_token) + 1;
            }
            return h;
        };
        auto fetch_pos = [&](const TileHeader& h) -> int64_t {
            return (h.kind != kKindDone && lane < h.ntok) ? p.position_ids[h.first_token + lane] : 0;
        };
        // tile indices past total_tiles only ever compare as "done"; saturate instead of wrapping
        const uint32_t stride = gridDim.x;
        uint32_t tile = blockIdx.x;
        auto ahead = [&](uint32_t t, uint32_t k) {
            const uint64_t v = static_cast<uint64_t>(t) + static_cast<uint64_t>(k) * stride;
            return v > 0xffffffffull ? 0xffffffffu : static_cast<uint32_t>(v);
        };
        TileHeader cur = describe(tile);
        int64_t pos_cur = fetch_pos(cur);
        TileHeader nxt = describe(ahead(tile, 1));
        int64_t pos_nxt = fetch_pos(nxt);
        uint32_t issued = 0;
        bool ok = true;
        for (uint32_t it = 0;; ++it) {
            const TileHeader after = describe(ahead(tile, 2));  // positions are fetched two tiles ahead
            const int64_t pos_after = fetch_pos(after);
            const int s = it % STAGES;
            ok = mbar_wait(&empty[s], ((it / STAGES) & 1) ^ 1, abort_flag, p.wait_cycles);
            if (!ok) break;
            if (lane == 0) headers[s] = cur;
            if (cur.kind == kKindDone) {
                if (lane == 0) mbar_arrive(&full[s]);
                break;
            }
            uint8_t* stage = smem + s * L::kStageBytes;
            if (lane == 0) {
                const uint32_t row_bytes = static_cast<uint32_t>(cur.nrows) * kRowBytes;
                // self-test hook: for one chosen tile, announce 16 bytes that are never sent, so that the waits on this
                // stage run out (p.short_tile is 0xffffffff in every ordinary launch)
                const uint32_t never_sent = tile == p.short_tile ? 16u : 0u;
                mbar_arrive_expect_tx(&full[s], row_bytes + static_cast<uint32_t>(cur.ntok) * kCosSinRowBytes + never_sent);
                const uint8_t* src = (cur.kind == kKindQ ? p.q : p.kv) + static_cast<uint64_t>(cur.row0) * kRowBytes;
                bulk_load(stage, src, row_bytes, &full[s]);
            }
            __syncwarp();
            if (lane < cur.ntok)
                bulk_load(stage + L::kDataBytes + lane * kCosSinRowBytes, p.cos_sin + pos_cur * kRopeDim, kCosSinRowBytes,
                          &full[s]);
            issued = it + 1;
            tile = ahead(tile, 1);
            cur = nxt, pos_cur = pos_nxt;
            nxt = after, pos_nxt = pos_after;
        }
        if (!ok) {
            // gave up: let the copies already issued land before the CTA (and its shared memory) goes away
            const uint32_t first = issued > STAGES ? issued - STAGES : 0;
            for (uint32_t it = first; it < issued; ++it)
            {
                const long long start = clock64();
                while (!mbar_try_wait(&full[it % STAGES], (it / STAGES) & 1) && clock64() - start < p.wait_cycles) {
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------ storer
        if (lane == 0) {
            for (uint32_t it = 0;; ++it) {
                const int s = it % STAGES;
                const uint32_t parity = (it / STAGES) & 1;
                if (!mbar_wait(&full[s], parity, abort_flag, p.wait_cycles)) break;
                const TileHeader h = headers[s];
                if (h.kind == kKindDone) break;
                if (!mbar_wait(&done[s], parity, abort_flag, p.wait_cycles)) break;
                if (h.kind == kKindQ)
                    bulk_store(p.q + static_cast<uint64_t>(h.row0) * kRowBytes, smem + s * L::kStageBytes, static_cast<uint32_t>(h.nrows) * kRowBytes);
                bulk_commit();
                if (it >= PENDING) {
                    bulk_wait_read<PENDING>();  // the store of tile it-PENDING no longer reads its stage
                    mbar_arrive(&empty[(it - PENDING) % STAGES]);
                }
            }
            bulk_wait_all();
        }
    } else {
        // ------------------------------------------------------------ workers
        const int w = warp - 2;
        for (uint32_t it = 0;; ++it) {
            const int s = it % STAGES;
            if (!mbar_wait(&full[s], (it / STAGES) & 1, abort_flag, p.wait_cycles)) break;
            const TileHeader h = headers[s];
            if (h.kind == kKindDone) break;
            uint8_t* stage = smem + s * L::kStageBytes;
            const float* cs_stage = reinterpret_cast<const float*>(stage + L::kDataBytes);
            if (h.kind == kKindQ) {
#pragma unroll
                for (int i = w; i < TILE; i += WORKERS) {
                    if (i >= h.nrows) break;
                    // A/B/T layout out of shared memory: 16 + 16 (lanes < 24) + 4 bytes per lane
                    uint8_t* row = stage + i * kRowBytes;
                    uint4* row16 = reinterpret_cast<uint4*>(row);
                    uint32_t* tail4 = reinterpret_cast<uint32_t*>(row + 2 * kNopeDim);
                    float xa[8], xb[8];
                    unpack8(row16[lane], xa);
                    unpack8(lane < kFirstRopeLane ? row16[32 + lane] : make_uint4(0u, 0u, 0u, 0u), xb);
                    const uint32_t tail = tail4[lane];
                    const float r = row_inv_rms(xa, xb, tail, p.eps);
                    scale8(xa, r), scale8(xb, r);
                    const float* cs = cs_stage + fast_div(h.rem + i, p.heads_mul, p.heads_shift) * kRopeDim;
                    row16[lane] = pack8(xa);
                    if (lane < kFirstRopeLane) row16[32 + lane] = pack8(xb);
                    tail4[lane] = scale_rotate_pair(tail, r, cs[lane], cs[32 + lane]);
                }
                fence_async_smem();  // generic-proxy writes above -> visible to the bulk store
            } else {
                for (int i = w; i < h.nrows; i += WORKERS) {
                    const int64_t t = static_cast<int64_t>(h.row0) + i;
                    const int64_t slot = p.slot_mapping[t];
                    if (slot < 0) continue;
                    const uint4* row = reinterpret_cast<const uint4*>(stage + i * kRowBytes);
                    const uint4 a = row[lane], b = row[32 + lane];
                    float4 c = make_float4(0.f, 0.f, 0.f, 0.f), sn = c;
                    if (lane >= kFirstRopeLane) {
                        const float* cs = cs_stage + i * kRopeDim + 4 * (lane - kFirstRopeLane);
                        c = *reinterpret_cast<const float4*>(cs);
                        sn = *reinterpret_cast<const float4*>(cs + 32);
                    }
                    const int64_t block = slot / p.block_size, in_block = slot - block * p.block_size;
                    uint8_t* base = p.k_cache + block * p.block_stride;
                    kv_row_to_cache(a, b, lane, c, sn, base + in_block * kTokenDataBytes,
                                    base + p.block_size * kTokenDataBytes + in_block * kScaleBytes,
                                    p.cache_aligned16 != 0);
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&done[s]);
        }
    }
}

// Per-device set-up, done once per device however many host threads make their first call at the same time.
struct DeviceInfo {
    std::once_flag once;
    int sm_count = 0;
    cudaError_t status = cudaSuccess;
};
DeviceInfo g_devices[64];

template <int TILE, int STAGES, int WORKERS, int PENDING, int CTAS_PER_SM>
cudaError_t launch(const PrologueParams& p, cudaStream_t stream) {
    using L = BulkLayout<TILE, STAGES, WORKERS>;
    static_assert(L::kTotalBytes * CTAS_PER_SM <= 227 * 1024, "stages do not fit in shared memory");
    auto kernel = prologue_bulk_kernel<TILE, STAGES, WORKERS, PENDING, CTAS_PER_SM>;
    int dev = 0;
    cudaError_t err = cudaGetDevice(&dev);
    if (err != cudaSuccess) return err;
    if (dev < 0 || dev >= 64) return cudaErrorInvalidDevice;
    DeviceInfo& info = g_devices[dev];
    std::call_once(info.once, [&]() {
        info.status = cudaDeviceGetAttribute(&info.sm_count, cudaDevAttrMultiProcessorCount, dev);
        if (info.status == cudaSuccess)
            info.status = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kTotalBytes);
    });
    if (info.status != cudaSuccess) return info.status;
    if (info.sm_count <= 0) return cudaErrorInvalidDevice;
    const int64_t kv_tiles = (p.num_tokens_insert + TILE - 1) / TILE;
    const int64_t q_tiles = (p.num_tokens * p.num_heads + TILE - 1) / TILE;
    const int64_t total = kv_tiles + q_tiles;
    if (total == 0) return cudaSuccess;
    if (total >= 0xffffffffLL) return cudaErrorInvalidConfiguration;
    const int64_t resident = static_cast<int64_t>(info.sm_count) * CTAS_PER_SM;
    const int64_t grid = total < resident ? total : resident;
    kernel<<<static_cast<unsigned>(grid), L::kThreads, L::kTotalBytes, stream>>>(p, static_cast<uint32_t>(kv_tiles),
                                                                               static_cast<uint32_t>(total));
    count_launch();
    return cudaGetLastError();
}

}  // namespace

cudaError_t launch_prologue_bulk(const PrologueParams& p, cudaStream_t stream) {
#ifdef DSV4_BULK_TILE
    return launch<DSV4_BULK_TILE, DSV4_BULK_STAGES, DSV4_BULK_WORKERS, DSV4_BULK_PENDING, DSV4_BULK_CTAS_PER_SM>(p, stream);
#else
    return launch<16, 10, 16, 2, 1>(p, stream);
#endif
}

// Reads and clears the device-side error word of the current device (synchronises).
cudaError_t read_device_error(int* value) {
    int zero = 0;
    cudaError_t err = cudaMemcpyFromSymbol(value, g_device_error, sizeof(int));
    if (err != cudaSuccess) return err;
    return cudaMemcpyToSymbol(g_device_error, &zero, sizeof(int));
}

}  // namespace dsv4
