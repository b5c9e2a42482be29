// Fused pair im2col_histc: one translation unit per pair so that the variants compile in parallel.
#include "dl_host.cuh"

DEFINE_PAIR_(im2col_histc, IM2COL_, HISTC_)
