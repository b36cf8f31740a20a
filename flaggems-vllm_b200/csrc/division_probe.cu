// On-device check of the quantisers' division shortcut (ScaleDivider in dsv4_common.cuh), part of the aid library
// libdsv4_hbm_probe.so, not of the operator library.
//
// The CPU proof of the shortcut enumerates every (group maximum, value) pair for each of the three values the refined
// reciprocal can take; this kernel runs the device's own reciprocal - `rcp.approx` included, whose result no CPU can
// reproduce bit for bit - over the same pairs and counts the e4m3 bytes that differ from those of the IEEE quotient.
// For every non-negative finite bf16 amax (32640 of them): scale = RN(max(amax, eps) * RN(1/448)), and for every bf16
// value x with 0 <= x <= amax the byte of form 2 (two-term, scales up to 2^100 only) or form 3 (corrected product).
#include "../../include/dsv4_hbm_probe.h"
#include "dsv4_common.cuh"

namespace dsv4 {
namespace {

constexpr int kAmaxValues = 0x7f80;  // bf16 bit patterns of the non-negative finite values

template <bool TWO_TERM>
__global__ void __launch_bounds__(256) division_probe_kernel(float eps, unsigned long long* counts) {
    const int ia = blockIdx.x;  // one CTA per group maximum
    const float amax = __uint_as_float(static_cast<uint32_t>(ia) << 16);
    const float scale = __fmul_rn(fmaxf(amax, eps), 1.0f / 448.0f);
    const ScaleDivider<kDivideFast> by_scale(scale);
    unsigned long long pairs = 0, mismatches = 0, reciprocal_off = 0;
    if (!TWO_TERM || by_scale.allows_two_term()) {
        for (int ix = threadIdx.x; ix <= ia; ix += blockDim.x) {
            const float x = __uint_as_float(static_cast<uint32_t>(ix) << 16);
            const uint32_t got = pack_e4m3x4(by_scale.template quotient<TWO_TERM>(x), 0.f, 0.f, 0.f) & 0xffu;
            const uint32_t want = pack_e4m3x4(__fdiv_rn(x, scale), 0.f, 0.f, 0.f) & 0xffu;
            ++pairs;
            mismatches += got != want;
        }
    }
    if (threadIdx.x == 0) {
        // how far the refined reciprocal is from the correctly rounded one, in units in the last place
        const int d = static_cast<int>(__float_as_uint(by_scale.recip)) - static_cast<int>(__float_as_uint(__frcp_rn(scale)));
        reciprocal_off = (d < -1 || d > 1) ? 1 : 0;
    }
    atomicAdd(&counts[0], pairs);
    atomicAdd(&counts[1], mismatches);
    atomicAdd(&counts[2], reciprocal_off);
}

}  // namespace
}  // namespace dsv4

extern "C" int dsv4_division_probe(float eps, int form, unsigned long long* counts, void* cuda_stream) {
    if (!counts) return -1;
    if (form != 2 && form != 3) return -2;
    cudaStream_t stream = static_cast<cudaStream_t>(cuda_stream);
    if (form == 2) dsv4::division_probe_kernel<true><<<dsv4::kAmaxValues, 256, 0, stream>>>(eps, counts);
    else dsv4::division_probe_kernel<false><<<dsv4::kAmaxValues, 256, 0, stream>>>(eps, counts);
    return static_cast<int>(cudaGetLastError());
}
