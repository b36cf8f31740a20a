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
// One CTA per row, radix selection in two reads of the row (the second one out of L2):
//   1. histogram of a coarse, monotone 11-bit code of every value (top bits of its fp16 rounding, which spreads real
//      logits over hundreds of bins where the top bits of the fp32 pattern would hit a handful);
//   2. the bin holding the k-th largest value is located; values in higher bins are emitted straight away, the
//      values of that bin are collected in shared memory with their full 32-bit keys;
//   3. the collected candidates are reduced by a byte-wise radix selection in shared memory.
// A bin with more candidates than fit in shared memory (degenerate inputs: thousands of near-equal values) takes a
// slower route: three more histogram reads of the row on the bits of the fp32 key, then one emitting read.
// HBM traffic: the row once (4 bytes per value); top_k * 4 bytes written.
#include <cuda_fp16.h>

#include "dsv4_common.cuh"

namespace dsv4 {
namespace {

constexpr int kTopkThreads = 512;
constexpr int kBins = 2048;
constexpr int kCandidateCap = 4096;

struct TopkParams {
    const float* logits;
    int64_t stride0, stride1;
    int32_t* indices;  // [num_rows, top_k]
    int32_t num_rows, vocab, top_k;
    // decode
    const int32_t* seq_lens;
    int32_t next_n;
    // prefill
    const int32_t* row_starts;
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

template <bool DECODE>
__global__ void __launch_bounds__(kTopkThreads) topk_per_row_kernel(const TopkParams p) {
    __shared__ uint32_t hist[kBins];
    __shared__ uint2 cand[kCandidateCap];  // (order key, position)
    __shared__ uint32_t scratch[32];
    __shared__ uint32_t result[4];
    __shared__ uint32_t counters[4];  // 0: emitted, 1: candidates collected, 2: ties taken
    const int tid = threadIdx.x;
    const int row = blockIdx.x;
    int64_t start, end;
    if (DECODE) {
        start = 0;
        end = static_cast<int64_t>(p.seq_lens[row / p.next_n]) - p.next_n + row % p.next_n + 1;
    } else {
        start = p.row_starts[row];
        end = p.row_ends[row];
    }
    start = start < 0 ? 0 : start;
    end = end > p.vocab ? p.vocab : end;
    const int32_t len = end > start ? static_cast<int32_t>(end - start) : 0;
    const int32_t k = len < p.top_k ? len : p.top_k;
    int32_t* out = p.indices + static_cast<int64_t>(row) * p.top_k;
    for (int i = k + tid; i < p.top_k; i += kTopkThreads) out[i] = -1;
    if (len <= p.top_k) {  // everything is selected
        for (int i = tid; i < len; i += kTopkThreads) out[i] = i;
        return;
    }
    const float* x = p.logits + static_cast<int64_t>(row) * p.stride0 + start * p.stride1;
    const auto load = [&](int32_t i) { return __uint_as_float(ld_stream4(x + static_cast<int64_t>(i) * p.stride1)); };

    // 1. coarse histogram
    for (int i = tid; i < kBins; i += kTopkThreads) hist[i] = 0u;
    if (tid < 4) counters[tid] = 0u;
    __syncthreads();
    {
        int32_t i = tid;
        for (; i + 3 * kTopkThreads < len; i += 4 * kTopkThreads) {
            const float a = load(i), b = load(i + kTopkThreads), c = load(i + 2 * kTopkThreads), d = load(i + 3 * kTopkThreads);
            atomicAdd(&hist[coarse_bin(a)], 1u), atomicAdd(&hist[coarse_bin(b)], 1u);
            atomicAdd(&hist[coarse_bin(c)], 1u), atomicAdd(&hist[coarse_bin(d)], 1u);
        }
        for (; i < len; i += kTopkThreads) atomicAdd(&hist[coarse_bin(load(i))], 1u);
    }
    __syncthreads();
    const Threshold coarse = find_threshold(hist, static_cast<uint32_t>(k), scratch, result);
    const bool collect = coarse.count <= kCandidateCap && coarse.need < coarse.count;
    const bool take_all = coarse.need == coarse.count;  // the whole bin belongs to the top k

    // 2. emit everything above the bin (and the bin itself if it is taken whole); collect the bin's candidates
    {
        const auto visit = [&](int32_t i, float v) {
            const uint32_t c = coarse_bin(v);
            if (c > coarse.bin || (take_all && c == coarse.bin)) {
                out[atomicAdd(&counters[0], 1u)] = i;
            } else if (collect && c == coarse.bin) {
                cand[atomicAdd(&counters[1], 1u)] = make_uint2(order_key(__float_as_uint(v)), static_cast<uint32_t>(i));
            }
        };
        int32_t i = tid;
        for (; i + 3 * kTopkThreads < len; i += 4 * kTopkThreads) {
            const float a = load(i), b = load(i + kTopkThreads), c = load(i + 2 * kTopkThreads), d = load(i + 3 * kTopkThreads);
            visit(i, a), visit(i + kTopkThreads, b), visit(i + 2 * kTopkThreads, c), visit(i + 3 * kTopkThreads, d);
        }
        for (; i < len; i += kTopkThreads) visit(i, load(i));
    }
    __syncthreads();
    if (take_all) return;

    uint32_t need = coarse.need;  // how many of the bin's elements are still to be emitted
    uint32_t prefix = 0u, prefix_mask = 0u;
    if (collect) {
        // 3. byte-wise radix selection among the candidates in shared memory
        const uint32_t n_cand = coarse.count;
        for (int shift = 24; shift >= 0; shift -= 8) {
            for (int i = tid; i < kBins; i += kTopkThreads) hist[i] = 0u;
            __syncthreads();
            for (uint32_t i = tid; i < n_cand; i += kTopkThreads) {
                const uint32_t key = cand[i].x;
                if ((key & prefix_mask) == prefix) atomicAdd(&hist[(key >> shift) & 0xffu], 1u);
            }
            __syncthreads();
            const Threshold t = find_threshold(hist, need, scratch, result);
            prefix |= t.bin << shift;
            prefix_mask |= 0xffu << shift;
            need = t.need;
        }
        // prefix is now the key of the k-th largest value; `need` of the candidates equal to it are taken
        for (uint32_t i = tid; i < n_cand; i += kTopkThreads) {
            const uint2 e = cand[i];
            if (e.x > prefix || (e.x == prefix && atomicAdd(&counters[2], 1u) < need)) out[atomicAdd(&counters[0], 1u)] = static_cast<int32_t>(e.y);
        }
        return;
    }

    // Slow route: the bin is too crowded for shared memory.  Radix selection on the fp32 key over the row itself,
    // restricted to the elements of the bin: bits 31-21, 20-10, 9-0.
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
    if (seq_lens) topk_per_row_kernel<true><<<static_cast<unsigned>(num_rows), kTopkThreads, 0, stream>>>(p);
    else topk_per_row_kernel<false><<<static_cast<unsigned>(num_rows), kTopkThreads, 0, stream>>>(p);
    count_launch();
    return cudaGetLastError();
}

}  // namespace dsv4
