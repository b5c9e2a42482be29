"""ctypes binding of `libhfuse_b200.so` (the C ABI declared in include/hfuse_b200.h).

The library must have been built (``python -m hfuse_b200.build``); loading
fails loudly otherwise — there is no CPU or PyTorch fallback for any entry point.
"""
from __future__ import annotations

import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libhfuse_b200.so")

HFUSE_MAX_HITS = 256
HFUSE_NOALLOC_MAX_CHANNELS = 1024

_p, _i, _f = C.c_void_p, C.c_int, C.c_float
_i64, _u64, _u32, _sz = C.c_int64, C.c_uint64, C.c_uint32, C.c_size_t

# parameter lists, in the order of the HFUSE_*_PARAMS macros
IM2COL = [_p, _i, _i, _i, _i, _i, _i, _i, _i, _i, _i, _i, _i, _p]
MAXPOOL = [_p, _i, _i, _i, _i, _i, _i, _i, _i, _i, _i, _i, _i, _i, _i, _p, _p]
BNSTATS = [_p, _i, _i, _i, _f, _p, _p, _p, _p, _sz]
UPSAMPLE = [_p, _i, _i, _i, _i, _i, _i, _i, _p]
HISTC = [_p, _i64, _i, _f, _f, _p]
SEARCH = [C.c_char_p, _u64, _u64, C.c_char_p, _p]                 # header80, start, count, target32, hits
ETHASH = [_p, _u32, C.c_char_p, _u64, _u64, C.c_char_p, _p]       # dag, items, header_hash32, start, count, target32, hits

_PARAMS = {"im2col": IM2COL, "maxpool": MAXPOOL, "bnstats": BNSTATS, "upsample": UPSAMPLE, "histc": HISTC,
           "blake256": SEARCH, "sha256d": SEARCH, "sia": SEARCH, "ethash": ETHASH}

DL_SOLO = {"im2col": "hfuse_im2col_f32", "maxpool": "hfuse_maxpool2d_f32", "bnstats": "hfuse_bnstats_f32",
           "upsample": "hfuse_upsample_bilinear2d_f32", "histc": "hfuse_histc_f32"}
# pair name -> (first half, second half); order as in the reference's configs/ml_fusion.yaml
DL_PAIRS = {
    "im2col_maxpool": ("im2col", "maxpool"), "im2col_bnstats": ("im2col", "bnstats"),
    "im2col_histc": ("im2col", "histc"), "im2col_upsample": ("im2col", "upsample"),
    "maxpool_bnstats": ("maxpool", "bnstats"), "maxpool_upsample": ("maxpool", "upsample"),
    "histc_maxpool": ("histc", "maxpool"), "histc_upsample": ("histc", "upsample"),
    "upsample_bnstats": ("upsample", "bnstats"), "histc_bnstats": ("histc", "bnstats"),
}
CRYPTO_SOLO = {"blake256": "hfuse_blake256_search", "sha256d": "hfuse_sha256d_search",
               "sia": "hfuse_sia_blake2b_search", "ethash": "hfuse_ethash_search"}
# order as in the reference's configs/crypto_fusion.yaml
CRYPTO_PAIRS = {
    "ethash_blake256": ("ethash", "blake256"), "sha256d_ethash": ("sha256d", "ethash"),
    "sia_ethash": ("sia", "ethash"), "blake256_sha256d": ("blake256", "sha256d"),
    "blake256_sia": ("blake256", "sia"), "sha256d_sia": ("sha256d", "sia"),
}


class Hits(C.Structure):
    """Mirror of `hfuse_hits`."""
    _fields_ = [("count", C.c_uint32), ("reserved", C.c_uint32),
                ("nonce", C.c_uint64 * HFUSE_MAX_HITS),
                ("mix", (C.c_uint32 * 8) * HFUSE_MAX_HITS)]


def exported_symbols() -> list[str]:
    """Every function include/hfuse_b200.h declares."""
    names = list(DL_SOLO.values()) + [f"hfuse_{p}_f32" for p in DL_PAIRS]
    names += list(CRYPTO_SOLO.values()) + [f"hfuse_{p}_search" for p in CRYPTO_PAIRS]
    names += ["hfuse_exchange_create", "hfuse_exchange_local_handle", "hfuse_exchange_connect",
              "hfuse_exchange_status", "hfuse_exchange_clear_status", "hfuse_exchange_destroy", "hfuse_exchange_local_pointer",
              "hfuse_exchange_connect_pointers", "hfuse_exchange_set_timeout", "hfuse_bnstats_allreduce_f32",
              "hfuse_upsample_bnstats_allreduce_f32"]
    names += ["hfuse_ethash_make_cache", "hfuse_ethash_generate_dag"]
    names += ["hfuse_comm_unique_id", "hfuse_comm_create", "hfuse_comm_destroy", "hfuse_bnstats_allreduce_nccl_f64",
              "hfuse_histc_allreduce_counts", "hfuse_dag_broadcast", "hfuse_blake256_sha256d_search_sharded",
              "hfuse_sia_ethash_search_sharded"]
    names += ["hfuse_maxpool2d_backward_f32", "hfuse_bn_backward_f32", "hfuse_maxpool_backward_bn_backward_f32"]
    names += ["hfuse_error_string", "hfuse_version", "hfuse_bnstats_workspace_bytes", "hfuse_bnstats_noalloc_f32",
              "hfuse_bnstats_finalize_f64", "hfuse_hits_reset", "hfuse_hash_batch", "hfuse_tune_set",
              "hfuse_tune_describe", "hfuse_tune_default", "hfuse_tune_set_share", "hfuse_tune_option", "hfuse_xoshiro256ss_fill", "hfuse_int32_probe", "hfuse_hbm_probe", "hfuse_hbm_probe_bulk", "hfuse_shard_range"]
    return names


class HfuseError(RuntimeError):
    def __init__(self, code: int, where: str):
        self.code = code
        super().__init__(f"{where}: {error_string(code)} ({code})")


_lib = None


def lib() -> C.CDLL:
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python -m hfuse_b200.build` "
            "(there is no fallback path without the CUDA library)")
    L = C.CDLL(LIB_PATH)
    for key, sym in DL_SOLO.items():
        fn = getattr(L, sym)
        fn.restype, fn.argtypes = _i, _PARAMS[key] + [_p]
    for name, (a, b) in DL_PAIRS.items():
        fn = getattr(L, f"hfuse_{name}_f32")
        fn.restype, fn.argtypes = _i, _PARAMS[a] + _PARAMS[b] + [_p]
    for key, sym in CRYPTO_SOLO.items():
        fn = getattr(L, sym)
        fn.restype, fn.argtypes = _i, _PARAMS[key] + [_p]
    for name, (a, b) in CRYPTO_PAIRS.items():
        fn = getattr(L, f"hfuse_{name}_search")
        fn.restype, fn.argtypes = _i, _PARAMS[a] + _PARAMS[b] + [_p]
    L.hfuse_error_string.restype, L.hfuse_error_string.argtypes = C.c_char_p, [_i]
    L.hfuse_version.restype, L.hfuse_version.argtypes = _i, []
    L.hfuse_bnstats_workspace_bytes.restype, L.hfuse_bnstats_workspace_bytes.argtypes = _sz, [_i, _i, _i]
    L.hfuse_bnstats_finalize_f64.restype = _i
    L.hfuse_bnstats_finalize_f64.argtypes = [_p, _i, _f, _p, _p, _p]
    L.hfuse_bnstats_noalloc_f32.restype = _i
    L.hfuse_bnstats_noalloc_f32.argtypes = [_p, _i, _i, _i, _f, _p, _p, _p, _p]
    L.hfuse_exchange_create.restype, L.hfuse_exchange_create.argtypes = _i, [_i, _i, _i, C.POINTER(_p)]
    L.hfuse_exchange_local_handle.restype, L.hfuse_exchange_local_handle.argtypes = _i, [_p, C.c_char_p]
    L.hfuse_exchange_connect.restype, L.hfuse_exchange_connect.argtypes = _i, [_p, C.c_char_p]
    L.hfuse_exchange_status.restype, L.hfuse_exchange_status.argtypes = _i, [_p, C.POINTER(_i)]
    L.hfuse_exchange_clear_status.restype, L.hfuse_exchange_clear_status.argtypes = _i, [_p, _p]
    L.hfuse_exchange_local_pointer.restype, L.hfuse_exchange_local_pointer.argtypes = _i, [_p, C.POINTER(C.c_void_p)]
    L.hfuse_exchange_connect_pointers.restype = _i
    L.hfuse_exchange_connect_pointers.argtypes = [_p, C.POINTER(C.c_void_p)]
    L.hfuse_exchange_set_timeout.restype, L.hfuse_exchange_set_timeout.argtypes = _i, [_p, _u64]
    L.hfuse_exchange_destroy.restype, L.hfuse_exchange_destroy.argtypes = _i, [_p]
    L.hfuse_bnstats_allreduce_f32.restype, L.hfuse_bnstats_allreduce_f32.argtypes = _i, BNSTATS + [_p, _p]
    L.hfuse_upsample_bnstats_allreduce_f32.restype = _i
    L.hfuse_upsample_bnstats_allreduce_f32.argtypes = UPSAMPLE + BNSTATS + [_p, _p]
    MPB = [_p, _p] + [_i] * 14 + [_p]
    BNB = [_p, _p, _i, _i, _i, _p, _p, _p, _p, _p, _p]
    L.hfuse_maxpool2d_backward_f32.restype, L.hfuse_maxpool2d_backward_f32.argtypes = _i, MPB + [_p]
    L.hfuse_bn_backward_f32.restype, L.hfuse_bn_backward_f32.argtypes = _i, BNB + [_p]
    L.hfuse_maxpool_backward_bn_backward_f32.restype = _i
    L.hfuse_maxpool_backward_bn_backward_f32.argtypes = MPB + BNB + [_p]
    L.hfuse_comm_unique_id.restype, L.hfuse_comm_unique_id.argtypes = _i, [C.c_char_p]
    L.hfuse_comm_create.restype, L.hfuse_comm_create.argtypes = _i, [_i, _i, C.c_char_p, C.POINTER(_p)]
    L.hfuse_comm_destroy.restype, L.hfuse_comm_destroy.argtypes = _i, [_p]
    L.hfuse_bnstats_allreduce_nccl_f64.restype = _i
    L.hfuse_bnstats_allreduce_nccl_f64.argtypes = [_p, _p, _i, _f, _p, _p, _p]
    L.hfuse_histc_allreduce_counts.restype, L.hfuse_histc_allreduce_counts.argtypes = _i, [_p, _p, _i, _p]
    L.hfuse_dag_broadcast.restype, L.hfuse_dag_broadcast.argtypes = _i, [_p, _p, _sz, _i, _p]
    L.hfuse_blake256_sha256d_search_sharded.restype = _i
    L.hfuse_blake256_sha256d_search_sharded.argtypes = SEARCH + SEARCH + [_i, _i, _p]
    L.hfuse_sia_ethash_search_sharded.restype = _i
    L.hfuse_sia_ethash_search_sharded.argtypes = SEARCH + ETHASH + [_i, _i, _p]
    L.hfuse_ethash_make_cache.restype, L.hfuse_ethash_make_cache.argtypes = _i, [C.c_char_p, _u32, _p]
    L.hfuse_ethash_generate_dag.restype = _i
    L.hfuse_ethash_generate_dag.argtypes = [_p, _u32, _p, _u32, _u32, _p]
    L.hfuse_hits_reset.restype, L.hfuse_hits_reset.argtypes = _i, [_p, _p]
    L.hfuse_hash_batch.restype = _i
    L.hfuse_hash_batch.argtypes = [_i, C.c_char_p, _p, _u32, _u64, _u32, _p, _p, _p]
    L.hfuse_tune_set.restype, L.hfuse_tune_set.argtypes = _i, [C.c_char_p, _i, _i]
    L.hfuse_tune_describe.restype, L.hfuse_tune_describe.argtypes = _i, [C.c_char_p, _i, C.c_char_p, _sz]
    L.hfuse_tune_set_share.restype, L.hfuse_tune_set_share.argtypes = _i, [C.c_char_p, _i]
    L.hfuse_tune_option.restype, L.hfuse_tune_option.argtypes = _i, [C.c_char_p, _i]
    L.hfuse_tune_default.restype, L.hfuse_tune_default.argtypes = _i, [C.c_char_p]
    L.hfuse_xoshiro256ss_fill.restype, L.hfuse_xoshiro256ss_fill.argtypes = None, [_u64, _p, _sz]
    L.hfuse_shard_range.restype = _i
    L.hfuse_shard_range.argtypes = [_u64, _i, _i, C.POINTER(C.c_uint64), C.POINTER(C.c_uint64)]
    L.hfuse_hbm_probe.restype, L.hfuse_hbm_probe.argtypes = _i, [_p, _sz, _p, _sz, _p]
    L.hfuse_hbm_probe_bulk.restype, L.hfuse_hbm_probe_bulk.argtypes = _i, [_p, _sz, _p, _sz, _p]
    L.hfuse_int32_probe.restype, L.hfuse_int32_probe.argtypes = _i, [_i, _u32, _p, C.POINTER(C.c_uint64), _p]
    _lib = L
    return L


def error_string(code: int) -> str:
    return lib().hfuse_error_string(code).decode()


def check(code: int, where: str) -> None:
    if code != 0:
        raise HfuseError(code, where)


def tune_set(name: str, variant: int = -1, blocks_per_sm: int = 0) -> None:
    check(lib().hfuse_tune_set(name.encode(), variant, blocks_per_sm), f"tune_set({name})")


def tune_set_share(name: str, permille: int = -1) -> None:
    check(lib().hfuse_tune_set_share(name.encode(), permille), f"tune_set_share({name})")


def tune_option(name: str, value: int) -> None:
    check(lib().hfuse_tune_option(name.encode(), value), f"tune_option({name})")


def tune_default(name: str) -> str:
    """Descriptor ("T1:T2:minBlocks") of the compiled default variant of a kernel or pair."""
    v = lib().hfuse_tune_default(name.encode())
    check(min(v, 0), f"tune_default({name})")
    return tune_variants(name.removesuffix("_wide"))[v]      # "<exchange pair>_wide": its default beyond four ranks


def tune_variants(name: str) -> list[str]:
    buf = C.create_string_buffer(64)
    n = lib().hfuse_tune_describe(name.encode(), 0, buf, 64)
    check(min(n, 0), f"tune_describe({name})")
    out = []
    for v in range(n):
        lib().hfuse_tune_describe(name.encode(), v, buf, 64)
        out.append(buf.value.decode())
    return out
