// Fused pair maxpool_upsample: one translation unit per pair so that the variants compile in parallel.
#include "dl_host.cuh"

DEFINE_PAIR_(maxpool_upsample, MAXPOOL_, UPSAMPLE_)
