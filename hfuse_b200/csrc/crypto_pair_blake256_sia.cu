// Fused pair blake256_sia: one translation unit per pair so that the variants compile in parallel.
#include "crypto_host.cuh"

DEFINE_CPAIR_(blake256_sia, BLAKE_, SIA_)
