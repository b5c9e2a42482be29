// Fused pair maxpool_bnstats: one translation unit per pair so that the variants compile in parallel.
#include "dl_host.cuh"

DEFINE_PAIR_(maxpool_bnstats, MAXPOOL_, BNSTATS_)
