// Fused pair histc_maxpool: one translation unit per pair so that the variants compile in parallel.
#include "dl_host.cuh"

DEFINE_PAIR_(histc_maxpool, HISTC_, MAXPOOL_)
