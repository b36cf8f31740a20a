/*
 * C ABI of libdsv4_hbm_probe.so: measurement and test aids, built separately from the operator library
 * (libdsv4_prologue.so, include/dsv4_prologue.h) so that the product library exports operators only.
 * The benchmark uses it to measure, on the GPU at hand, the streaming rates the fused kernels are compared with.
 */
#ifndef DSV4_HBM_PROBE_H
#define DSV4_HBM_PROBE_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/*
 * Bandwidth probe with the prologue's q access pattern and no arithmetic, over `rows` rows of
 * 1 KiB starting at `buffer` (16-byte aligned): mode 0 reads every row and writes it back in
 * place, mode 1 only reads, mode 2 only writes (the buffer's contents are overwritten), mode 3 reads
 * every row and writes 512 bytes per row behind the rows (the buffer then holds rows * 1536 bytes;
 * 2 read : 1 write, the mix of the narrowing sibling operators).  Used by
 * bench.py to measure, on the GPU at hand, the ceiling the fused kernel is compared with.
 * Returns 0, a negative code (-1 NULL buffer, -2 bad mode or size, -3 buffer not 16-byte aligned) or a cudaError_t.
 * No counterpart in the reference.
 */
int dsv4_hbm_probe(int mode, void* buffer, int64_t rows, void* cuda_stream);

/*
 * On-device check of the division shortcut the quantisers use for fp32 scales (product with a refined approximate
 * reciprocal; form 2 = two-term, scales up to 2^100, form 3 = corrected product, any scale).  For every non-negative
 * finite bf16 group maximum and every bf16 value up to it, with scale = max(amax, eps) / 448 as the operators form it,
 * adds to counts[0] the pairs examined, to counts[1] those whose e4m3 byte differs from that of the IEEE quotient and
 * to counts[2] the scales whose refined reciprocal is more than one unit in the last place from the correctly rounded
 * one.  `counts` is caller-allocated device memory of three 64-bit words that the caller has zeroed.  A test aid: the
 * CPU proof covers the three values such a reciprocal can take, this runs the device's own.
 * Returns 0, -1 (NULL counts), -2 (unknown form) or a cudaError_t.  No counterpart in the reference.
 */
int dsv4_division_probe(float eps, int form, unsigned long long* counts, void* cuda_stream);


#ifdef __cplusplus
}
#endif

#endif /* DSV4_HBM_PROBE_H */
