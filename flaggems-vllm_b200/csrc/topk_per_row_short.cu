// The top-k selection kernel compiled a second time with 256 threads per CTA, for launches whose rows are at most
// 8192 values wide: such rows spend their time in the short phases between barriers, and CTAs of 8 warps overlap
// those better than CTAs of 16 (measured 7-26 % faster on 2048 ... 8192 wide rows; slower on everything wider).
#define DSV4_TOPK_THREADS 256
#define launch_topk_per_row launch_topk_per_row_short
#include "topk_per_row.cu"
