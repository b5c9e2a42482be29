// Fused pair im2col_maxpool: one translation unit per pair so that the variants compile in parallel.
#include "dl_host.cuh"

DEFINE_PAIR_(im2col_maxpool, IM2COL_, MAXPOOL_)
