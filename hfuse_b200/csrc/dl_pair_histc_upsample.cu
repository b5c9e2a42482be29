// Fused pair histc_upsample: one translation unit per pair so that the variants compile in parallel.
#include "dl_host.cuh"

DEFINE_PAIR_(histc_upsample, HISTC_, UPSAMPLE_)
