// Fused pair blake256_sha256d: one translation unit per pair so that the variants compile in parallel.
#include "crypto_host.cuh"

DEFINE_CPAIR_(blake256_sha256d, BLAKE_, SHA_)
