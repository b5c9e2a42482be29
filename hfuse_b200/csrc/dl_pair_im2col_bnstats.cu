// Fused pair im2col_bnstats: one translation unit per pair so that the variants compile in parallel.
#include "dl_host.cuh"

DEFINE_PAIR_(im2col_bnstats, IM2COL_, BNSTATS_)
