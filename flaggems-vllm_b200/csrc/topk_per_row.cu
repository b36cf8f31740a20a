// top_k_per_row_decode / top_k_per_row_prefill: the indices of the top_k largest logits of every row inside the
// row's valid range, the selection step of the sparse indexer between its logits and the index bookkeeping.
// Reference: src/flaggems_vllm/ops/top_k_per_row_decode.py:1263-1399, src/flaggems_vllm/ops/top_k_per_row_prefill.py
// (wrapper `top_k_per_row_prefill`), and their torch statements tests/test_top_k_per_row_decode.py:111-124,
// tests/test_top_k_per_row_prefill.py:80-99:
//   row i, range [start_i, end_i): k = min(top_k, end_i - start_i); indices[i, :k] = positions (relative to start_i) of
//   the k largest values, in any order, ties broken arbitrarily; indices[i, k:] = -1.
//   decode:  start_i = 0, end_i = seq_lens[i / next_n] - next_n + i % next_n + 1
//   prefill: start_i = row_starts[i], end_i = row_ends[i]
//
// One CTA per row, or a thread-block cluster of 2 / 4 / 8 CTAs for long rows.  Values are ranked by a coarse, monotone 11-bit code (top bits of the fp16 rounding of the value,
// which spreads real logits over hundreds of bins where the top bits of the fp32 pattern would hit a handful) and,
// inside a bin, by the order-preserving 32-bit key of their fp32 pattern.
//   Fast route, ONE read of the row: a sample of the row (128 runs of 32 values) gives a bin b0 above which k values
//   plus four standard deviations are expected; the row is streamed once and every value in a bin >= b0 is put
//   into shared memory with its key and position; if at least k and at most kCandidateCap values were collected, a
//   radix selection in shared memory finishes the job.  In a cluster every CTA streams its share of the row and hands
//   its candidates to the first CTA through distributed shared memory (two hardware cluster barriers, no spinning).
//   Histogram route, two reads (the second mostly out of L2), when the sample misjudged the row or k is too large for
//   the candidate buffer: 1. histogram of the coarse code over the whole row, 2. the bin of the k-th largest value is
//   located, values in higher bins are emitted, the values of that bin are collected in shared memory, 3. radix
//   selection among them.
//   A bin with more values than fit in shared memory (degenerate inputs: thousands of near-equal values) takes three
//   more histogram reads of the row on the bits of the fp32 key, then one emitting read.
// The result does not depend on the route; the sample only decides how fast it is reached.
// HBM traffic on the fast route: the row once (4 bytes per value); top_k * 4 bytes written.
#include <cooperative_groups.h>
#include <cuda_fp16.h>

#include <mutex>

#include "dsv4_common.cuh"

namespace dsv4 {
namespace {

namespace cg = cooperative_groups;

#ifndef DSV4_TOPK_THREADS
#define DSV4_TOPK_THREADS 512
#endif
constexpr int kTopkThreads = DSV4_TOPK_THREADS;
constexpr int kBins = 2048;
constexpr int kCandidateCap = 8192;  // 64 KiB of (key, position) pairs in dynamic shared memory
constexpr int kSampleChunks = 128;  // x 32 values
constexpr int kCountingMax = kBins / 2;  // candidates of one bin ranked by counting (they are kept where the histogram was)

struct TopkParams {
    const float* logits;
    int64_t stride0, stride1;
    int32_t* indices;  // [num_rows, top_k]
    int32_t num_rows, vocab, top_k;
    uint32_t pair_capacity;  // (key, position) pairs the dynamic shared memory of this launch holds
    // decode
    const int32_t* seq_lens;
    int32_t next_n;
    // prefill
    const int32_t* row_starts;  // null: every range starts at 0
    const int32_t* row_ends;
};

// Unsigned key with the order of the float values (negative values below positive ones, -0 below +0).
__device__ __forceinline__ uint32_t order_key(uint32_t bits) { return (bits & 0x80000000u) ? ~bits : bits | 0x80000000u; }

// Coarse monotone code: the top 11 bits of the order key of the value rounded to fp16.
__device__ __forceinline__ uint32_t coarse_bin(float x) {
    const uint32_t h = __half_as_ushort(__float2half_rn(x));
    const uint32_t key = (h & 0x8000u) ? (~h & 0xffffu) : (h | 0x8000u);
    return key >> 5;
}

struct Threshold {
    uint32_t bin;    // the bin holding the k-th largest element
    uint32_t need;   // how many elements of that bin belong to the top k
    uint32_t count;  // how many elements that bin holds
};

// The bin, counted from the top, in which the running count reaches `want` (1 <= want <= total of hist).
// All threads call it; hist has kBins entries; `scratch` holds 32 words.  Ends with a barrier.
__device__ __forceinline__ Threshold find_threshold(const uint32_t* hist, uint32_t want, uint32_t* scratch, uint32_t* result) {
    constexpr int kPerThread = kBins / kTopkThreads;  // 4 bins per thread, thread 0 owns the highest ones
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    uint32_t local[kPerThread], sum = 0;
#pragma unroll
    for (int j = 0; j < kPerThread; ++j) {
        local[j] = hist[kBins - 1 - (tid * kPerThread + j)];
        sum += local[j];
    }
    uint32_t incl = sum;
#pragma unroll
    for (int m = 1; m < 32; m <<= 1) {
        const uint32_t up = __shfl_up_sync(0xffffffffu, incl, m);
        if (lane >= m) incl += up;
    }
    if (lane == 31) scratch[warp] = incl;
    __syncthreads();
    if (warp == 0) {
        uint32_t w = lane < kTopkThreads / 32 ? scratch[lane] : 0u, wi = w;
#pragma unroll
        for (int m = 1; m < 32; m <<= 1) {
            const uint32_t up = __shfl_up_sync(0xffffffffu, wi, m);
            if (lane >= m) wi += up;
        }
        scratch[lane] = wi - w;  // exclusive prefix of the warp totals
    }
    __syncthreads();
    uint32_t above = scratch[warp] + incl - sum;  // elements in bins higher than this thread's
    if (above < want && want <= above + sum) {
#pragma unroll
        for (int j = 0; j < kPerThread; ++j) {
            if (above < want && want <= above + local[j]) {
                result[0] = kBins - 1 - (tid * kPerThread + j);
                result[1] = want - above;
                result[2] = local[j];
            }
            above += local[j];
        }
    }
    __syncthreads();
    Threshold t;
    t.bin = result[0], t.need = result[1], t.count = result[2];
    __syncthreads();
    return t;
}

// Histogram increment shared by the lanes of a warp that hit the same bin (degenerate inputs put a whole warp
// into one bin, which plain shared-memory atomics would serialise).
__device__ __forceinline__ void add_aggregated(uint32_t* hist, uint32_t bin, bool active) {
    const uint32_t mask = __ballot_sync(0xffffffffu, active);
    if (!active) return;
    const uint32_t peers = __match_any_sync(mask, bin);
    if ((threadIdx.x & 31) == __ffs(peers) - 1) atomicAdd(&hist[bin], __popc(peers));
}

// The `want` largest of the n candidates (key, position) in shared memory; their positions are appended to out
// through counters[0], ties at the smallest selected key through counters[2].  Radix selection in digits of up to
// 11 bits on key - min(key), starting at the highest bit in which the candidates differ at all (they share sign,
// exponent and leading mantissa bits, which a selection on fixed bit positions would waste passes and atomic
// conflicts on).
__device__ __forceinline__ void select_in_shared(const uint2* cand, uint32_t n, uint32_t want, uint32_t* hist, uint32_t* scratch,
                                                 uint32_t* result, uint32_t* counters, int32_t* out) {
    const int tid = threadIdx.x;
    if (want >= n) {
        for (uint32_t i = tid; i < n; i += kTopkThreads) out[atomicAdd(&counters[0], 1u)] = static_cast<int32_t>(cand[i].y);
        return;
    }
    // range of the keys
    if (tid == 0) result[0] = 0xffffffffu, result[1] = 0u;
    __syncthreads();
    uint32_t lo = 0xffffffffu, hi = 0u;
    for (uint32_t i = tid; i < n; i += kTopkThreads) {
        const uint32_t key = cand[i].x;
        lo = key < lo ? key : lo, hi = key > hi ? key : hi;
    }
    lo = __reduce_min_sync(0xffffffffu, lo), hi = __reduce_max_sync(0xffffffffu, hi);
    if ((tid & 31) == 0) atomicMin(&result[0], lo), atomicMax(&result[1], hi);
    __syncthreads();
    const uint32_t base = result[0], range = result[1] - result[0];
    __syncthreads();
    uint32_t need = want, prefix = 0u, prefix_mask = 0u;
    int top = 32 - __clz(range | 1u);  // bits of (key - base) that can be set
    while (top > 0) {
        const int shift = top > 11 ? top - 11 : 0;
        const uint32_t digit_mask = (1u << (top - shift)) - 1u;
        for (int i = tid; i < kBins; i += kTopkThreads) hist[i] = 0u;
        __syncthreads();
        for (uint32_t i = tid; i < n; i += kTopkThreads) {
            const uint32_t rel = cand[i].x - base;
            if ((rel & prefix_mask) == prefix) atomicAdd(&hist[(rel >> shift) & digit_mask], 1u);
        }
        __syncthreads();
        const Threshold t = find_threshold(hist, need, scratch, result);
        prefix |= t.bin << shift;
        prefix_mask |= digit_mask << shift;
        need = t.need;
        top = shift;
        if (t.need == t.count) break;  // every candidate with this prefix is taken: the lower bits do not matter
    }
    // keys above the prefix (on the bits examined) are in; `need` of those equal to it are in
    for (uint32_t i = tid; i < n; i += kTopkThreads) {
        const uint2 e = cand[i];
        const uint32_t rel_hi = (e.x - base) & prefix_mask;
        if (rel_hi > prefix || (rel_hi == prefix && atomicAdd(&counters[2], 1u) < need)) out[atomicAdd(&counters[0], 1u)] = static_cast<int32_t>(e.y);
    }
}

__device__ __forceinline__ uint32_t coarse_bin_of_key(uint32_t key) {  // key -> value -> bin
    return coarse_bin(__uint_as_float((key & 0x80000000u) ? key & 0x7fffffffu : ~key));
}

// The `want` largest of n candidates by counting: a candidate's rank is the number of candidates ahead of it in the
// total order (key descending, position ascending); one pass, no histogram.
__device__ __forceinline__ void rank_by_counting(const uint2* dense, uint32_t n, uint32_t want, uint32_t* counters, int32_t* out) {
    for (uint32_t a = threadIdx.x; a < n; a += kTopkThreads) {
        const uint2 e = dense[a];
        uint32_t ahead = 0u;
#pragma unroll 8
        for (uint32_t b = 0; b < n; ++b) {
            const uint2 o = dense[b];  // the same address for all lanes: a broadcast
            ahead += (o.x > e.x || (o.x == e.x && o.y < e.y)) ? 1u : 0u;
        }
        if (ahead < want) out[atomicAdd(&counters[0], 1u)] = static_cast<int32_t>(e.y);
    }
}

// The `want` largest of the n <= kCandidateCap candidates in `cand`, in two levels: a histogram of their coarse codes
// finds the bin of the want-th largest; candidates above it are emitted; those inside it are copied to where the
// histogram was and ranked by counting: a candidate's rank is the number of them ahead of it in the total order (key
// descending, position ascending).  A crowded bin goes to the radix selection instead.
// counters[1] must be zero on entry; `hist_ready` says that hist already holds the histogram.
__device__ __forceinline__ void select_two_level(const uint2* cand, uint32_t n, uint32_t want, uint32_t* hist, uint32_t* scratch,
                                                 uint32_t* result, uint32_t* counters, int32_t* out, bool hist_ready) {
    const int tid = threadIdx.x;
    if (!hist_ready) {
        for (int i = tid; i < kBins; i += kTopkThreads) hist[i] = 0u;
        __syncthreads();
        for (uint32_t i = tid; i < n; i += kTopkThreads) atomicAdd(&hist[coarse_bin_of_key(cand[i].x)], 1u);
        __syncthreads();
    }
    const Threshold coarse = find_threshold(hist, want, scratch, result);
    const bool take_all = coarse.need == coarse.count;
    if (!take_all && coarse.count > kCountingMax) {
        select_in_shared(cand, n, want, hist, scratch, result, counters, out);
        return;
    }
    uint2* dense = reinterpret_cast<uint2*>(hist);  // the histogram is no longer needed: kBins / 2 entries
    for (uint32_t i = tid; i < n; i += kTopkThreads) {
        const uint2 e = cand[i];
        const uint32_t c = coarse_bin_of_key(e.x);
        if (c > coarse.bin || (take_all && c == coarse.bin)) out[atomicAdd(&counters[0], 1u)] = static_cast<int32_t>(e.y);
        else if (c == coarse.bin) dense[atomicAdd(&counters[1], 1u)] = e;
    }
    __syncthreads();
    if (take_all) return;
    rank_by_counting(dense, coarse.count, coarse.need, counters, out);
}

template <bool DECODE>
__global__ void __launch_bounds__(kTopkThreads) topk_per_row_kernel(const TopkParams p) {
    __shared__ __align__(8) uint32_t hist[kBins];
    extern __shared__ uint2 cand[];  // kCandidateCap entries: (order key, position)
    __shared__ uint32_t scratch[32];
    __shared__ uint32_t result[4];
    __shared__ uint32_t counters[4];  // 0: emitted, 1: candidates collected, 2: ties taken
    cg::cluster_group cluster = cg::this_cluster();
    const uint32_t ctas = cluster.num_blocks(), rank = cluster.block_rank();  // the CTAs of a cluster share one row
    const int tid = threadIdx.x;
    const int row = blockIdx.x / ctas;
    int64_t start, end;
    if (DECODE) {
        start = 0;
        end = static_cast<int64_t>(p.seq_lens[row / p.next_n]) - p.next_n + row % p.next_n + 1;
    } else {
        start = p.row_starts ? p.row_starts[row] : 0;
        end = p.row_ends[row];
    }
    start = start < 0 ? 0 : start;
    end = end > p.vocab ? p.vocab : end;
    const int32_t len = end > start ? static_cast<int32_t>(end - start) : 0;
    const int32_t k = len < p.top_k ? len : p.top_k;
    int32_t* out = p.indices + static_cast<int64_t>(row) * p.top_k;
    // Everything up to the first cluster barrier depends on the row only, so the CTAs of a cluster leave together.
    if (rank == 0)
        for (int i = k + tid; i < p.top_k; i += kTopkThreads) out[i] = -1;
    if (len <= p.top_k) {  // everything is selected
        if (rank == 0)
            for (int i = tid; i < len; i += kTopkThreads) out[i] = i;
        return;
    }
    const float* x = p.logits + static_cast<int64_t>(row) * p.stride0 + start * p.stride1;
    const auto load = [&](int32_t i) { return __uint_as_float(ld_stream4(x + static_cast<int64_t>(i) * p.stride1)); };
    // Calls visit(position, value) for the elements [from, to) of the row; 16-byte loads where the layout allows.
    const auto for_each = [&](int32_t from, int32_t to, auto&& visit) {
        if (p.stride1 == 1) {
            int32_t head = from + static_cast<int32_t>(((16u - (reinterpret_cast<uintptr_t>(x + from) & 15u)) & 15u) >> 2);  // first 16-byte boundary
            head = head < to ? head : to;
            const int32_t vecs = (to - head) >> 2;
            const float* body = x + head;
            int32_t v = tid;
            for (; v + 3 * kTopkThreads < vecs; v += 4 * kTopkThreads) {  // four 16-byte loads per thread in flight
                uint4 q[4];
#pragma unroll
                for (int u = 0; u < 4; ++u) q[u] = ld_stream16(body + 4 * (v + u * kTopkThreads));
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    const int32_t i = head + 4 * (v + u * kTopkThreads);
                    visit(i, __uint_as_float(q[u].x)), visit(i + 1, __uint_as_float(q[u].y)), visit(i + 2, __uint_as_float(q[u].z)), visit(i + 3, __uint_as_float(q[u].w));
                }
            }
            for (; v < vecs; v += kTopkThreads) {
                const uint4 a = ld_stream16(body + 4 * v);
                const int32_t ia = head + 4 * v;
                visit(ia, __uint_as_float(a.x)), visit(ia + 1, __uint_as_float(a.y)), visit(ia + 2, __uint_as_float(a.z)), visit(ia + 3, __uint_as_float(a.w));
            }
            for (int32_t i = from + tid; i < head; i += kTopkThreads) visit(i, load(i));
            for (int32_t i = head + 4 * vecs + tid; i < to; i += kTopkThreads) visit(i, load(i));
        } else {
            for (int32_t i = from + tid; i < to; i += kTopkThreads) visit(i, load(i));
        }
    };

    const bool fast = 2 * k + 512 <= kCandidateCap;
    if (rank != 0 && (!fast || len <= kCandidateCap)) return;  // these rows are handled by the first CTA alone
    for (int i = tid; i < kBins; i += kTopkThreads) hist[i] = 0u;
    if (tid < 4) counters[tid] = 0u;
    __syncthreads();

    // ---- fast route -------------------------------------------------------------------------------------------
    if (fast && len <= kCandidateCap) {
        // The whole row fits into shared memory (keys only: a value's position is its place in the buffer): one read
        // fills it and the coarse histogram; values above the bin of the k-th largest are emitted, the few inside it
        // are copied to where the histogram was and ranked by counting.
        uint32_t* keys = reinterpret_cast<uint32_t*>(cand);
        for_each(0, len, [&](int32_t i, float v) {
            keys[i] = order_key(__float_as_uint(v));
            atomicAdd(&hist[coarse_bin(v)], 1u);
        });
        __syncthreads();
        const Threshold coarse = find_threshold(hist, static_cast<uint32_t>(k), scratch, result);
        const bool take_all = coarse.need == coarse.count;
        if (take_all || coarse.count <= kCountingMax) {
            uint2* dense = reinterpret_cast<uint2*>(hist);
            for (int32_t i = tid; i < len; i += kTopkThreads) {
                const uint32_t key = keys[i];
                const uint32_t c = coarse_bin_of_key(key);
                if (c > coarse.bin || (take_all && c == coarse.bin)) out[atomicAdd(&counters[0], 1u)] = i;
                else if (c == coarse.bin) dense[atomicAdd(&counters[1], 1u)] = make_uint2(key, static_cast<uint32_t>(i));
            }
            __syncthreads();
            if (!take_all) rank_by_counting(dense, coarse.count, coarse.need, counters, out);
            return;
        }
        // a crowded bin: over to the histogram route, which has the histogram it needs already
    } else if (fast) {
        // every CTA of the cluster takes the same sample, hence the same b0: candidates are the values in bins >= b0
        // the sample: kSampleChunks runs of 32 consecutive values (one 128-byte line each) spread evenly over the row
        const int32_t stride = (len / kSampleChunks) & ~31;  // len > kCandidateCap, so the runs do not overlap
        for (int32_t j = tid; j < kSampleChunks * 32; j += kTopkThreads) atomicAdd(&hist[coarse_bin(load((j >> 5) * stride + (j & 31)))], 1u);
        __syncthreads();
        // rank inside the sample that stands for k values of the row, plus four standard deviations of that count
        const float mean = static_cast<float>(k) * (kSampleChunks * 32) / static_cast<float>(len);
        const uint32_t sample_rank = static_cast<uint32_t>(mean + 4.0f * sqrtf(mean)) + 3u;
        const uint32_t b0 = find_threshold(hist, sample_rank < kSampleChunks * 32u ? sample_rank : kSampleChunks * 32u, scratch, result).bin;
        cluster.sync();  // the first CTA's counters are zero before anybody reserves space in its buffer
        // this CTA's share of the row, a multiple of 4 elements so that the 16-byte loads stay aligned
        const int32_t share = (((len + static_cast<int32_t>(ctas) - 1) / static_cast<int32_t>(ctas)) + 3) & ~3;
        const int32_t from = static_cast<int32_t>(rank) * share < len ? static_cast<int32_t>(rank) * share : len;
        const int32_t to = from + share < len ? from + share : len;
        for_each(from, to, [&](int32_t i, float v) {
            if (coarse_bin(v) >= b0) {
                const uint32_t at = atomicAdd(&counters[1], 1u);
                if (at < kCandidateCap) cand[at] = make_uint2(order_key(__float_as_uint(v)), static_cast<uint32_t>(i));
            }
        });
        __syncthreads();
        if (rank != 0) {
            // hand the candidates over to the first CTA through distributed shared memory
            const uint32_t mine = counters[1];
            if (tid == 0) result[3] = atomicAdd(cluster.map_shared_rank(&counters[1], 0), mine);
            __syncthreads();
            const uint32_t at = result[3];
            if (mine <= kCandidateCap && at + mine <= kCandidateCap) {
                uint2* remote = cluster.map_shared_rank(cand, 0);
                for (uint32_t j = tid; j < mine; j += kTopkThreads) remote[at + j] = cand[j];
            }
        }
        cluster.sync();  // all candidates have arrived
        if (rank != 0) return;
        const uint32_t collected = counters[1];
        if (collected >= static_cast<uint32_t>(k) && collected <= kCandidateCap) {
            __syncthreads();
            if (tid == 0) counters[1] = 0u;
            select_two_level(cand, collected, static_cast<uint32_t>(k), hist, scratch, result, counters, out, false);
            return;
        }
        // the sample misjudged the row: the first CTA starts over on the histogram route
        __syncthreads();
        for (int i = tid; i < kBins; i += kTopkThreads) hist[i] = 0u;
        if (tid < 4) counters[tid] = 0u;
        __syncthreads();
    }

    // ---- histogram route --------------------------------------------------------------------------------------
    if (!(fast && len <= kCandidateCap)) {  // (a short row arrives with its histogram)
        for_each(0, len, [&](int32_t, float v) { atomicAdd(&hist[coarse_bin(v)], 1u); });
        __syncthreads();
    }
    const Threshold coarse = find_threshold(hist, static_cast<uint32_t>(k), scratch, result);
    const bool collect = coarse.count <= p.pair_capacity && coarse.need < coarse.count;
    const bool take_all = coarse.need == coarse.count;  // the whole bin belongs to the top k
    // emit everything above the bin (and the bin itself if it is taken whole); collect the bin's candidates
    for_each(0, len, [&](int32_t i, float v) {
        const uint32_t c = coarse_bin(v);
        if (c > coarse.bin || (take_all && c == coarse.bin)) {
            out[atomicAdd(&counters[0], 1u)] = i;
        } else if (collect && c == coarse.bin) {
            cand[atomicAdd(&counters[1], 1u)] = make_uint2(order_key(__float_as_uint(v)), static_cast<uint32_t>(i));
        }
    });
    __syncthreads();
    if (take_all) return;
    if (collect) {
        select_in_shared(cand, coarse.count, coarse.need, hist, scratch, result, counters, out);
        return;
    }

    // Slow route: the bin is too crowded for shared memory.  Radix selection on the fp32 key over the row itself,
    // restricted to the elements of the bin: bits 31-21, 20-10, 9-0.
    uint32_t need = coarse.need, prefix = 0u, prefix_mask = 0u;
    const int shifts[3] = {21, 10, 0};
    const uint32_t widths[3] = {11, 11, 10};
    for (int pass = 0; pass < 3; ++pass) {
        for (int i = tid; i < kBins; i += kTopkThreads) hist[i] = 0u;
        __syncthreads();
        const int32_t padded = (len + 31) & ~31;  // whole warps stay together for the aggregated increment
        for (int32_t i = tid; i < padded; i += kTopkThreads) {
            bool active = false;
            uint32_t bin = 0u;
            if (i < len) {
                const float v = load(i);
                const uint32_t key = order_key(__float_as_uint(v));
                active = coarse_bin(v) == coarse.bin && (key & prefix_mask) == prefix;
                bin = (key >> shifts[pass]) & ((1u << widths[pass]) - 1u);
            }
            add_aggregated(hist, bin, active);
        }
        __syncthreads();
        const Threshold t = find_threshold(hist, need, scratch, result);
        prefix |= t.bin << shifts[pass];
        prefix_mask |= ((1u << widths[pass]) - 1u) << shifts[pass];
        need = t.need;
    }
    for (int32_t i = tid; i < len; i += kTopkThreads) {
        const float v = load(i);
        if (coarse_bin(v) != coarse.bin) continue;
        const uint32_t key = order_key(__float_as_uint(v));
        if (key > prefix || (key == prefix && atomicAdd(&counters[2], 1u) < need)) out[atomicAdd(&counters[0], 1u)] = i;
    }
}

}  // namespace

cudaError_t launch_topk_per_row(const float* logits, int64_t stride0, int64_t stride1, int32_t* indices, int64_t num_rows, int vocab,
                                int top_k, const int32_t* seq_lens, int next_n, const int32_t* row_starts, const int32_t* row_ends,
                                cudaStream_t stream) {
    if (num_rows == 0 || top_k == 0) return cudaSuccess;
    TopkParams p{};
    p.logits = logits, p.stride0 = stride0, p.stride1 = stride1, p.indices = indices;
    p.num_rows = static_cast<int32_t>(num_rows), p.vocab = vocab, p.top_k = top_k;
    p.seq_lens = seq_lens, p.next_n = next_n, p.row_starts = row_starts, p.row_ends = row_ends;
    constexpr size_t kDynamicBytes = sizeof(uint2) * kCandidateCap;
    // rows that fit into the buffer as a whole keep 4-byte keys only: more CTAs per SM for the many-short-rows case
    const size_t dynamic_bytes = vocab <= kCandidateCap ? sizeof(uint32_t) * static_cast<size_t>(vocab > 256 ? vocab : 256) : kDynamicBytes;
    // per-device set-up, once per device however many host threads make their first call at the same time
    struct DeviceSetup {
        std::once_flag once;
        cudaError_t status = cudaSuccess;
        int sms = 0;
    };
    static DeviceSetup setups[64];
    int dev = 0;
    cudaError_t err = cudaGetDevice(&dev);
    if (err != cudaSuccess) return err;
    if (dev < 0 || dev >= 64) return cudaErrorInvalidDevice;
    DeviceSetup& setup = setups[dev];
    std::call_once(setup.once, [&]() {
        setup.status = cudaFuncSetAttribute(topk_per_row_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(kDynamicBytes));
        if (setup.status == cudaSuccess)
            setup.status = cudaFuncSetAttribute(topk_per_row_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(kDynamicBytes));
        if (setup.status == cudaSuccess) setup.status = cudaDeviceGetAttribute(&setup.sms, cudaDevAttrMultiProcessorCount, dev);
    });
    if (setup.status != cudaSuccess) return setup.status;
    // CTAs per row: long rows are shared by a cluster (shorter streaming time per row, no straggling rows at the
    // end of the grid); the candidates meet in the first CTA's shared memory.
    // Only while the grid would not fill the GPU otherwise (about 3 CTAs per SM are resident): with many rows the
    // repeated sample and the barriers cost more than the shorter rows win.
    const int sms = setup.sms;
    unsigned ctas = vocab >= 131072 ? 8u : vocab >= 65536 ? 4u : vocab >= 32768 ? 2u : 1u;
    while (ctas > 1 && num_rows * ctas > 3LL * sms) ctas >>= 1;
    if (num_rows * ctas > 0x7fffffffLL) return cudaErrorInvalidConfiguration;
    cudaLaunchConfig_t config = {};
    config.gridDim = dim3(static_cast<unsigned>(num_rows * ctas)), config.blockDim = dim3(kTopkThreads);
    config.dynamicSmemBytes = dynamic_bytes, config.stream = stream;
    p.pair_capacity = static_cast<uint32_t>(dynamic_bytes / sizeof(uint2));
    cudaLaunchAttribute attribute[1];
    attribute[0].id = cudaLaunchAttributeClusterDimension;
    attribute[0].val.clusterDim.x = ctas, attribute[0].val.clusterDim.y = 1, attribute[0].val.clusterDim.z = 1;
    config.attrs = attribute, config.numAttrs = 1;
    err = seq_lens ? cudaLaunchKernelEx(&config, topk_per_row_kernel<true>, p) : cudaLaunchKernelEx(&config, topk_per_row_kernel<false>, p);
    if (err != cudaSuccess) return err;
    count_launch();
    return cudaGetLastError();
}

}  // namespace dsv4
