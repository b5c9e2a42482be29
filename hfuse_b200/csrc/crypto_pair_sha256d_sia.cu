// Fused pair sha256d_sia: one translation unit per pair so that the variants compile in parallel.
#include "crypto_host.cuh"

DEFINE_CPAIR_(sha256d_sia, SHA_, SIA_)
