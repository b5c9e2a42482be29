// Fused pair upsample_bnstats: one translation unit per pair so that the variants compile in parallel.
#include "dl_host.cuh"

DEFINE_PAIR_(upsample_bnstats, UPSAMPLE_, BNSTATS_)
