// Fused pair histc_bnstats: one translation unit per pair so that the variants compile in parallel.
#include "dl_host.cuh"

DEFINE_PAIR_(histc_bnstats, HISTC_, BNSTATS_)
