"""hfuse_b200 — horizontally fused CUDA kernel pairs for NVIDIA B200 (sm_100a).

Hand-written replacements for the fused kernels that aoli-al/HFuse emits:
the deep-learning pairs of its configs/ml_fusion.yaml and the nonce-search
pairs of its configs/crypto_fusion.yaml, behind the C ABI declared in
include/hfuse_b200.h.  `ops` is the Python call harness for the DL pairs,
`crypto` the one for the hash searches, `sharding` the multi-GPU host logic
and `workloads` the seeded synthetic inputs.
"""
__all__ = ["ops", "crypto", "sharding", "workloads", "build"]
