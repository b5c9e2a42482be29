"""The C-ABI library loads without a GPU and exports every symbol the public header declares."""
import ctypes
import os
import re

import numpy as np

from conftest import ROOT
from hfuse_b200 import _lib


def _declared_in_header():
    text = open(os.path.join(ROOT, "include", "hfuse_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"HFUSE_API\s+[\w\s\*]+?\b(hfuse_\w+)\s*\(", text)))


def test_every_declared_symbol_is_exported():
    declared = _declared_in_header()
    assert len(declared) >= 30
    L = ctypes.CDLL(_lib.LIB_PATH)
    for name in declared:
        assert hasattr(L, name), name
    assert sorted(_lib.exported_symbols()) == declared


def test_error_strings_and_version():
    assert _lib.lib().hfuse_version() >= 100
    assert _lib.error_string(0) == "ok"
    assert "aligned" in _lib.error_string(-2)


def test_tuning_table():
    for name in list(_lib.DL_SOLO) + list(_lib.DL_PAIRS) + list(_lib.CRYPTO_SOLO) + list(_lib.CRYPTO_PAIRS):
        v = _lib.tune_variants(name)
        assert len(v) >= 5
        assert _lib.tune_default(name) in v                            # the compiled default is one of them
        for d in v:
            t1, t2, mb = (int(x) for x in d.removesuffix(" queue").split(":"))   # "T:0:mb queue": work-queue form of a search
            assert t1 % 32 == 0 and t2 % 32 == 0 and mb >= 1        # whole warps; the DL lists move in 128-thread steps
            if name in _lib.DL_SOLO or name in _lib.DL_PAIRS:
                assert t1 % 128 == 0 and t2 % 128 == 0              # like the reference's sweep
    assert _lib.lib().hfuse_tune_set(b"no_such_pair", 0, 0) == -7
    assert _lib.lib().hfuse_tune_default(b"no_such_pair") == -7
    assert _lib.tune_default("upsample_bnstats_allreduce") in _lib.tune_variants("upsample_bnstats_allreduce")
    assert _lib.tune_default("upsample_bnstats_allreduce_wide") in _lib.tune_variants("upsample_bnstats_allreduce")   # beyond four ranks
    assert _lib.lib().hfuse_tune_set(b"im2col_maxpool", 999, 0) < 0
    _lib.tune_set("im2col_maxpool", 1, 2)
    _lib.tune_set("im2col_maxpool", -1, 0)
    # the exchange pair has its own entry (same variant list as the DL pairs) and a share knob
    assert _lib.tune_variants("upsample_bnstats_allreduce") == _lib.tune_variants("upsample_bnstats")
    L = _lib.lib()
    assert L.hfuse_tune_set_share(b"upsample_bnstats_allreduce", 250) == 0
    assert L.hfuse_tune_set_share(b"upsample_bnstats_allreduce", -1) == 0
    assert L.hfuse_tune_set_share(b"upsample_bnstats_allreduce", 1001) == -1
    assert L.hfuse_tune_set_share(b"upsample_bnstats", 100) == -7
    assert L.hfuse_tune_set_share(None, 100) == -1
    # exchange objects: argument checks that need no device
    assert L.hfuse_exchange_create(0, 0, 4, None) == -1
    assert L.hfuse_exchange_set_timeout(None, 1) == -1
    assert L.hfuse_exchange_connect_pointers(None, None) == -1


def test_bad_arguments_are_rejected_before_any_launch():
    L = _lib.lib()
    # null pointers / bad shapes: checked on the host, so no GPU is needed
    assert L.hfuse_im2col_f32(None, 1, 1, 4, 4, 3, 3, 1, 1, 1, 1, 1, 1, None, None) == -1
    assert L.hfuse_im2col_f32(16, 1, 1, 4, 4, 9, 9, 0, 0, 1, 1, 1, 1, 16, None) == -1      # kernel too large
    assert L.hfuse_im2col_f32(20, 1, 1, 4, 4, 3, 3, 1, 1, 1, 1, 1, 1, 16, None) == -2      # misaligned
    assert L.hfuse_histc_f32(16, 8, 4, 1.0, 1.0, 16, None) == -1                           # empty range
    assert L.hfuse_maxpool2d_f32(16, 1, 1, 4, 4, 9, 9, 2, 2, 2, 2, 0, 0, 1, 1, 16, 16, None) == -1
    assert L.hfuse_bnstats_f32(16, 0, 1, 1, 1e-5, 16, 16, None, None, 0, None) == -1
    tgt = bytes(32)
    assert L.hfuse_sha256d_search(bytes(80), 0, (1 << 32) + 1, tgt, 16, None) == -3        # beyond the nonce space
    assert L.hfuse_ethash_search(None, 0, bytes(32), 0, 1, tgt, 16, None) == -1


def test_host_generator_matches_oracle():
    from hfuse_b200 import workloads
    from oracle import crypto as OC
    assert np.array_equal(workloads.xoshiro_bytes(3, 4097), OC.xoshiro_bytes(3, 4097))
    c3 = workloads.config3()
    assert len(c3["blake_header"]) == 80 and len(c3["sha_header"]) == 80
    assert int.from_bytes(c3["target"], "big") == 2 ** 224


def test_fused_search_needs_two_different_hit_records_and_a_count_that_fits_the_queue():
    L = _lib.lib()
    hdr, target = bytes(80), bytes(32)
    rec, rec2 = 4096, 8192          # never dereferenced: the checks come before any CUDA call
    assert L.hfuse_blake256_sha256d_search(hdr, 0, 1 << 20, target, rec, hdr, 0, 1 << 20, target, rec, None) == -1
    assert L.hfuse_blake256_sia_search(hdr, 0, 1 << 20, target, rec, hdr, 0, (1 << 61) + 1, target, rec2, None) == -3
    assert L.hfuse_blake256_sia_search(hdr, 0, (1 << 32) + 1, target, rec, hdr, 0, 1 << 20, target, rec2, None) == -3
    assert L.hfuse_exchange_clear_status(None, None) == -1
    assert L.hfuse_tune_option(b"im2col_store_path", 2) == -1
    assert L.hfuse_tune_option(b"nothing", 1) == -7
    assert L.hfuse_tune_option(b"im2col_store_path", 0) == 0
    assert L.hfuse_tune_option(b"im2col_store_path", -1) == 0        # back to the compiled choice per kernel / pair
    assert L.hfuse_tune_option(b"exchange_pair_pool", 1) == 0
    assert L.hfuse_tune_option(b"exchange_pair_pool", -1) == 0
    assert L.hfuse_tune_option(b"bnstats_load_path", 1) == 0
    assert L.hfuse_tune_option(b"bnstats_load_path", -1) == 0
    assert L.hfuse_tune_option(b"histc_load_path", 1) == 0
    assert L.hfuse_tune_option(b"histc_load_path", -1) == 0


def test_ops_refuse_cpu_tensors():
    import pytest
    import torch
    from hfuse_b200 import ops
    with pytest.raises(RuntimeError, match="no CPU path"):
        ops.im2col(torch.zeros(1, 1, 4, 4), 3, 1)


def test_torch_extension_registers_every_pair_and_refuses_cpu_tensors():
    import pytest
    import torch
    from hfuse_b200 import torch_ops  # noqa: F401
    for name in list(_lib.DL_PAIRS) + ["im2col", "max_pool2d_with_indices", "batch_norm_stats", "upsample_bilinear2d",
                                       "histc"]:
        assert hasattr(torch.ops.hfuse_b200, name), name
    with pytest.raises(RuntimeError, match="no CPU path"):
        torch.ops.hfuse_b200.histc(torch.zeros(4), 4, 0.0, 1.0)


def test_public_header_is_valid_c_and_cpp(tmp_path):
    import subprocess
    hdr = os.path.join(ROOT, "include", "hfuse_b200.h")
    for lang, std in (("c", "-std=c99"), ("c++", "-std=c++17")):
        src = tmp_path / ("t." + ("c" if lang == "c" else "cpp"))
        src.write_text(f'#include "{hdr}"\nint main(void) {{ return (int)sizeof(hfuse_hits) == 0; }}\n')
        r = subprocess.run(["/usr/bin/gcc" if lang == "c" else "/usr/bin/g++", std, "-Wall", "-Werror", "-fsyntax-only",
                            str(src)], capture_output=True, text=True)
        assert r.returncode == 0, r.stderr
