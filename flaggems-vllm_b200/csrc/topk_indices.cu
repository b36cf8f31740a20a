// Index bookkeeping of the DeepSeek-V4 sparse attention, the two integer operators next to the cache reader:
//
// compute_global_topk_indices_and_lens (src/flaggems_vllm/ops/
//   deepseek_v4_attention_compute_global_topk_indices_and_lens.py:49-167): a token's top-k positions inside
//   its request (int32, negative = empty) become slots of the paged cache,
//   slot = block_table[req, pos / block_size] * block_size + pos % block_size, empty entries stay -1;
//   lens[token] = number of non-negative entries, or 0 when the token is marked invalid.
//
// combine_topk_swa_indices (src/flaggems_vllm/ops/deepseek_v4_attention_combine_topk_swa_indices.py:30-164):
//   per query token one row [compressed top-k entries | sliding-window entries | -1 padding] of indices into
//   the gathered key buffer, and its number of valid entries.
//
// Both are pure int32 streaming work: about one row read and one row written per token.
#include "dsv4_common.cuh"

namespace dsv4 {
namespace {

struct GlobalTopkParams {
    const int32_t* local;  // [T, topk], row stride in elements
    int64_t local_stride;
    const int32_t* token_to_req;  // [T]
    const int32_t* block_table;
    int64_t block_table_stride;
    const int32_t* is_valid;  // [T] or null (every token valid)
    int32_t* global;          // [T, topk]
    int64_t global_stride;
    int32_t* lens;  // [T]
    int64_t num_tokens;
    int32_t topk, block_size;
    int32_t bs_shift;  // log2(block_size) or -1
    uint32_t bs_mul, bs_mul_shift;
};

__device__ __forceinline__ int32_t to_slot(const GlobalTopkParams& p, const int32_t* table_row, int32_t local, int32_t* count) {
    if (local < 0) return -1;
    ++*count;
    const uint32_t u = static_cast<uint32_t>(local);
    const uint32_t block = p.bs_shift >= 0 ? u >> p.bs_shift : fast_div(u, p.bs_mul, p.bs_mul_shift);
    const int32_t in_block = static_cast<int32_t>(u - block * static_cast<uint32_t>(p.block_size));
    return __ldg(table_row + block) * p.block_size + in_block;
}

// One warp per token.  VEC: rows are 16-byte aligned and topk is a multiple of 4, so a lane moves 4 entries at a time.
template <int WARPS, bool VEC>
__global__ void __launch_bounds__(WARPS * 32) global_topk_kernel(const GlobalTopkParams p) {
    const int lane = threadIdx.x & 31;
    const int64_t t = static_cast<int64_t>(blockIdx.x) * WARPS + (threadIdx.x >> 5);
    if (t >= p.num_tokens) return;
    const int32_t* table_row = p.block_table + static_cast<int64_t>(__ldg(p.token_to_req + t)) * p.block_table_stride;
    const int32_t* in = p.local + t * p.local_stride;
    int32_t* out = p.global + t * p.global_stride;
    int32_t count = 0;
    if (VEC) {
        for (int c = 4 * lane; c < p.topk; c += 256) {
            // two chunks of 4 in flight per lane
            const bool second = c + 128 < p.topk;
            const uint4 a = ld_stream16(in + c);
            const uint4 b = second ? ld_stream16(in + c + 128) : make_uint4(0u, 0u, 0u, 0u);
            uint4 ra, rb;
            ra.x = to_slot(p, table_row, a.x, &count), ra.y = to_slot(p, table_row, a.y, &count);
            ra.z = to_slot(p, table_row, a.z, &count), ra.w = to_slot(p, table_row, a.w, &count);
            st_stream16(out + c, ra);
            if (second) {
                rb.x = to_slot(p, table_row, b.x, &count), rb.y = to_slot(p, table_row, b.y, &count);
                rb.z = to_slot(p, table_row, b.z, &count), rb.w = to_slot(p, table_row, b.w, &count);
                st_stream16(out + c + 128, rb);
            }
        }
    } else {
        for (int c = lane; c < p.topk; c += 32) out[c] = to_slot(p, table_row, in[c], &count);
    }
#pragma unroll
    for (int m = 16; m > 0; m >>= 1) count += __shfl_xor_sync(0xffffffffu, count, m);
    if (lane == 0) p.lens[t] = (p.is_valid == nullptr || __ldg(p.is_valid + t) != 0) ? count : 0;
}

struct CombineParams {
    const int32_t* topk;  // [T, topk_width], row stride in elements
    int64_t topk_stride;
    const int32_t* query_start_loc;  // [R + 1]
    const int32_t* seq_lens;         // [R]
    const int32_t* gather_lens;      // [R]
    int32_t* combined;               // [T, combined_width]
    int64_t combined_stride;
    int32_t* lens;  // [T]
    int32_t num_reqs, num_tokens;
    int32_t topk_width, combined_width;
    int32_t window, compress_ratio, top_k, m, n;
    int32_t search_steps;
    uint32_t cr_mul, cr_shift;
};

// One warp per query token.  VEC: rows 16-byte aligned and widths multiples of 4.
template <int WARPS, bool VEC>
__global__ void __launch_bounds__(WARPS * 32) combine_topk_swa_kernel(const CombineParams p) {
    const int lane = threadIdx.x & 31;
    const int32_t token = static_cast<int32_t>(blockIdx.x * WARPS + (threadIdx.x >> 5));
    if (token >= p.num_tokens) return;
    // request of the token: the last b with query_start_loc[b] - query_start_loc[0] <= token
    const int32_t base = __ldg(p.query_start_loc);
    int32_t left = 0, right = p.num_reqs + 1;
    for (int32_t s = 0; s < p.search_steps; ++s) {
        const int32_t mid = (left + right) >> 1;
        const bool before = mid <= p.num_reqs && __ldg(p.query_start_loc + mid) - base <= token;
        left = before ? mid + 1 : left;
        right = before ? right : mid;
    }
    const int32_t b = left - 1;
    if (b < 0 || b >= p.num_reqs) return;  // a row no request covers: not written, as in the reference
    const int32_t query_start = __ldg(p.query_start_loc + b) - base, query_end = __ldg(p.query_start_loc + b + 1) - base;
    if (token >= query_end) return;
    const int32_t seq_len = __ldg(p.seq_lens + b);
    const int32_t pos = seq_len - (query_end - query_start) + (token - query_start);
    const int32_t gather_start = seq_len - __ldg(p.gather_lens + b);
    // floor((pos + 1) / compress_ratio), also for a negative numerator
    const int32_t num = pos + 1;
    const int32_t quot = num >= 0 ? static_cast<int32_t>(fast_div(static_cast<uint32_t>(num), p.cr_mul, p.cr_shift))
                                  : -static_cast<int32_t>(fast_div(static_cast<uint32_t>(-num) + p.compress_ratio - 1, p.cr_mul, p.cr_shift));
    const int32_t topk_len = quot < p.top_k ? quot : p.top_k;
    const int32_t swa_len = num < p.window ? num : p.window;
    const int32_t valid_len = topk_len + swa_len;
    const int32_t shift = p.m * b;
    // column c of the window part holds swa_first + c
    const int32_t swa_first = shift + p.n + pos - swa_len + 1 - gather_start - topk_len;
    const int32_t* in = p.topk + static_cast<int64_t>(token) * p.topk_stride;
    int32_t* out = p.combined + static_cast<int64_t>(token) * p.combined_stride;
    const auto entry = [&](int32_t c, int32_t loaded) -> int32_t {
        return c < topk_len ? loaded + shift : (c < valid_len ? swa_first + c : -1);
    };
    if (VEC) {
        for (int32_t c = 4 * lane; c < p.combined_width; c += 128) {
            uint4 v = make_uint4(0u, 0u, 0u, 0u);
            if (c < topk_len) v = ld_stream16(in + c);  // stays inside the row: c + 4 <= topk_width because topk_len <= topk_width
            uint4 r;
            r.x = entry(c, v.x), r.y = entry(c + 1, v.y), r.z = entry(c + 2, v.z), r.w = entry(c + 3, v.w);
            st_stream16(out + c, r);
        }
    } else {
        for (int32_t c = lane; c < p.combined_width; c += 32) out[c] = entry(c, c < topk_len ? in[c] : 0);
    }
    if (lane == 0) p.lens[token] = valid_len;
}

}  // namespace

cudaError_t launch_global_topk(const int32_t* local, int64_t local_stride, const int32_t* token_to_req, const int32_t* block_table,
                               int64_t block_table_stride, const int32_t* is_valid, int32_t* global, int64_t global_stride,
                               int32_t* lens, int64_t num_tokens, int topk, int block_size, cudaStream_t stream) {
    if (num_tokens == 0) return cudaSuccess;
    constexpr int WARPS = 4;
    GlobalTopkParams p{};
    p.local = local, p.local_stride = local_stride, p.token_to_req = token_to_req, p.block_table = block_table;
    p.block_table_stride = block_table_stride, p.is_valid = is_valid, p.global = global, p.global_stride = global_stride;
    p.lens = lens, p.num_tokens = num_tokens, p.topk = topk, p.block_size = block_size;
    p.bs_shift = pow2_shift(block_size);
    make_fast_divisor(static_cast<uint32_t>(block_size), &p.bs_mul, &p.bs_mul_shift);
    const int64_t grid = (num_tokens + WARPS - 1) / WARPS;
    if (grid > 0x7fffffffLL) return cudaErrorInvalidConfiguration;
    const auto addr = [](const void* q) { return reinterpret_cast<uintptr_t>(q); };
    const bool vec = topk % 4 == 0 && local_stride % 4 == 0 && global_stride % 4 == 0 && addr(local) % 16 == 0 && addr(global) % 16 == 0;
    if (vec) global_topk_kernel<WARPS, true><<<static_cast<unsigned>(grid), WARPS * 32, 0, stream>>>(p);
    else global_topk_kernel<WARPS, false><<<static_cast<unsigned>(grid), WARPS * 32, 0, stream>>>(p);
    count_launch();
    return cudaGetLastError();
}

cudaError_t launch_combine_topk_swa(const int32_t* topk_indices, int64_t topk_stride, int topk_width, const int32_t* query_start_loc,
                                    const int32_t* seq_lens, const int32_t* gather_lens, int32_t* combined, int64_t combined_stride,
                                    int combined_width, int32_t* lens, int64_t num_reqs, int64_t num_tokens, int window,
                                    int compress_ratio, int top_k, int m, int n, cudaStream_t stream) {
    if (num_tokens == 0 || num_reqs == 0) return cudaSuccess;
    constexpr int WARPS = 4;
    CombineParams p{};
    p.topk = topk_indices, p.topk_stride = topk_stride, p.query_start_loc = query_start_loc, p.seq_lens = seq_lens;
    p.gather_lens = gather_lens, p.combined = combined, p.combined_stride = combined_stride, p.lens = lens;
    p.num_reqs = static_cast<int32_t>(num_reqs), p.num_tokens = static_cast<int32_t>(num_tokens);
    p.topk_width = topk_width, p.combined_width = combined_width;
    p.window = window, p.compress_ratio = compress_ratio, p.top_k = top_k, p.m = m, p.n = n;
    p.search_steps = 0;
    for (int64_t span = num_reqs + 1; span > 0; span >>= 1) ++p.search_steps;
    make_fast_divisor(static_cast<uint32_t>(compress_ratio), &p.cr_mul, &p.cr_shift);
    const int64_t grid = (num_tokens + WARPS - 1) / WARPS;
    if (grid > 0x7fffffffLL) return cudaErrorInvalidConfiguration;
    const auto addr = [](const void* q) { return reinterpret_cast<uintptr_t>(q); };
    const bool vec = topk_width % 4 == 0 && combined_width % 4 == 0 && topk_stride % 4 == 0 && combined_stride % 4 == 0 &&
                     addr(topk_indices) % 16 == 0 && addr(combined) % 16 == 0;
    if (vec) combine_topk_swa_kernel<WARPS, true><<<static_cast<unsigned>(grid), WARPS * 32, 0, stream>>>(p);
    else combine_topk_swa_kernel<WARPS, false><<<static_cast<unsigned>(grid), WARPS * 32, 0, stream>>>(p);
    count_launch();
    return cudaGetLastError();
}

}  // namespace dsv4
