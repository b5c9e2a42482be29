// Fused pair sha256d_ethash: one translation unit per pair so that the variants compile in parallel.
#include "crypto_host.cuh"

DEFINE_CPAIR_(sha256d_ethash, SHA_, ETH_)
