// HBM ceiling probes with the access pattern of the prologue's q path and no arithmetic:
// every warp moves whole 1-KiB rows with 16-byte accesses, two rows per warp, 4 warps per CTA.
// They answer "how fast can this GPU stream N KiB rows in place / read-only / write-only",
// which is the bound the fused kernel is measured against next to the driver's copy figure.
//
// A measurement aid: built into its own library (libdsv4_hbm_probe.so, declared in include/dsv4_hbm_probe.h),
// not into the operator library.
#include "../../include/dsv4_hbm_probe.h"
#include "dsv4_common.cuh"

namespace dsv4 {
namespace {

constexpr int kProbeWarps = 4, kProbeRows = 2;

// mode 0: read a row and write it back in place (1 read : 1 write, like the prologue)
// mode 1: read only (rows are xor-folded; the result is stored only if it hits a magic value)
// mode 2: write only
// mode 3: read a row, write half as many bytes to a second region behind the rows (2 read : 1 write, the
//         mix of the epilogue quantiser and of the other narrowing operators)
template <int MODE>
__global__ void __launch_bounds__(kProbeWarps * 32) hbm_probe_kernel(uint8_t* buf, uint32_t rows, uint32_t* sink) {
    const int lane = threadIdx.x & 31;
    const uint32_t row0 = (blockIdx.x * kProbeWarps + (threadIdx.x >> 5)) * kProbeRows;
    uint4 a[kProbeRows], b[kProbeRows];
    uint32_t fold = 0;
#pragma unroll
    for (int i = 0; i < kProbeRows; ++i) {
        a[i] = b[i] = make_uint4(row0, lane, i, 0u);
        if (MODE != 2 && row0 + i < rows) {
            const uint8_t* row = buf + static_cast<uint64_t>(row0 + i) * kRowBytes;
            // mode 0 rewrites what it reads, so it must not use the non-coherent (read-only) path
            a[i] = MODE == 0 ? ld_inplace16(row + 16 * lane) : ld_stream16(row + 16 * lane);
            b[i] = MODE == 0 ? ld_inplace16(row + 512 + 16 * lane) : ld_stream16(row + 512 + 16 * lane);
        }
    }
#pragma unroll
    for (int i = 0; i < kProbeRows; ++i) {
        if (row0 + i >= rows) break;
        uint8_t* row = buf + static_cast<uint64_t>(row0 + i) * kRowBytes;
        if (MODE == 1) {
            fold ^= a[i].x ^ a[i].y ^ a[i].z ^ a[i].w ^ b[i].x ^ b[i].y ^ b[i].z ^ b[i].w;
        } else if (MODE == 3) {
            uint8_t* half_row = buf + static_cast<uint64_t>(rows) * kRowBytes + static_cast<uint64_t>(row0 + i) * (kRowBytes / 2);
            st_stream16(half_row + 16 * lane, make_uint4(a[i].x ^ b[i].x, a[i].y ^ b[i].y, a[i].z ^ b[i].z, a[i].w ^ b[i].w));
        } else {
            st_stream16(row + 16 * lane, a[i]);
            st_stream16(row + 512 + 16 * lane, b[i]);
        }
    }
    if (MODE == 1 && fold == 0x9e3779b9u && sink) *sink = fold;
}

cudaError_t launch_hbm_probe(int mode, uint8_t* buf, int64_t rows, uint32_t* sink, cudaStream_t stream) {
    if (rows == 0) return cudaSuccess;
    const unsigned grid = static_cast<unsigned>((rows + kProbeWarps * kProbeRows - 1) / (kProbeWarps * kProbeRows));
    const uint32_t n = static_cast<uint32_t>(rows);
    if (mode == 0) hbm_probe_kernel<0><<<grid, kProbeWarps * 32, 0, stream>>>(buf, n, sink);
    else if (mode == 1) hbm_probe_kernel<1><<<grid, kProbeWarps * 32, 0, stream>>>(buf, n, sink);
    else if (mode == 3) hbm_probe_kernel<3><<<grid, kProbeWarps * 32, 0, stream>>>(buf, n, sink);
    else hbm_probe_kernel<2><<<grid, kProbeWarps * 32, 0, stream>>>(buf, n, sink);
    return cudaGetLastError();
}

}  // namespace
}  // namespace dsv4

extern "C" int dsv4_hbm_probe(int mode, void* buffer, int64_t rows, void* cuda_stream) {
    if (mode < 0 || mode > 3) return -2;
    if (rows < 0 || rows >= (1LL << 31)) return -2;
    if (rows == 0) return 0;
    if (!buffer) return -1;
    if (reinterpret_cast<uintptr_t>(buffer) & 15u) return -3;
    return static_cast<int>(dsv4::launch_hbm_probe(mode, static_cast<uint8_t*>(buffer), rows, nullptr, static_cast<cudaStream_t>(cuda_stream)));
}
