// Fused pair ethash_blake256: one translation unit per pair so that the variants compile in parallel.
#include "crypto_host.cuh"

DEFINE_CPAIR_(ethash_blake256, ETH_, BLAKE_)
