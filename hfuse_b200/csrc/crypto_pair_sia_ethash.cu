// Fused pair sia_ethash: one translation unit per pair so that the variants compile in parallel.
#include "crypto_host.cuh"

DEFINE_CPAIR_(sia_ethash, SIA_, ETH_)
