/*
 * C ABI of libdsv4_hbm_probe.so: a measurement aid, built separately from the operator library
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


#ifdef __cplusplus
}
#endif

#endif /* DSV4_HBM_PROBE_H */
