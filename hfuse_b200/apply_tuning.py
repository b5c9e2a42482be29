"""Writes the result of `python bench.py --tune` into the compiled defaults.

    python bench.py --tune > tune.json          (on a B200)
    python -m hfuse_b200.apply_tuning tune.json (anywhere; then rebuild)

    torchrun --nproc-per-node N bench.py --gpus N --tune-share > share.json   (on N B200s)
    python -m hfuse_b200.apply_tuning --share share.json

The reference picks the split and register cap of each pair by rebuilding and
profiling every candidate (scripts/profile_and_collect_data.py:40-57); here all
candidates are compiled in, the sweep runs once, and only the default index per
kernel / pair changes.
"""
from __future__ import annotations

import json
import os
import re
import sys

from . import _lib

CSRC = os.path.join(os.path.dirname(os.path.abspath(__file__)), "csrc")


def apply(path: str, csrc: str = CSRC) -> None:
    with open(path) as f:
        text = f.read()
    res = json.loads(text[text.index("{"):])
    for inc, solos, pairs in (("dl_tuned.inc", _lib.DL_SOLO, _lib.DL_PAIRS),
                              ("crypto_tuned.inc", _lib.CRYPTO_SOLO, _lib.CRYPTO_PAIRS)):
        p = os.path.join(csrc, inc)
        src = open(p).read()
        for kind, names in (("Solo", solos), ("Pair", pairs)):
            for name in names:
                entry = res["solo" if kind == "Solo" else "pair"].get(name)
                if entry is None:
                    continue
                src, n = re.subn(rf"(kDefault{kind}_{name} = )\d+;", rf"\g<1>{entry['best']};", src)
                assert n == 1, name
                if "im2col_bulk" in entry:       # store path of the im2col role in this kernel / pair
                    src, n = re.subn(rf"(kIm2colBulk_{name} = )\d+;", rf"\g<1>{int(entry['im2col_bulk'])};", src)
                    assert n == 1, name
                if "histc_bulk" in entry:        # load path of the histogram role in this kernel / pair
                    src, n = re.subn(rf"(kHistcBulk_{name} = )\d+;", rf"\g<1>{int(entry['histc_bulk'])};", src)
                    assert n == 1, name
                if "bnstats_bulk" in entry:      # load path of the statistics role in this kernel / pair
                    src, n = re.subn(rf"(kBnStatsBulk_{name} = )\d+;", rf"\g<1>{int(entry['bnstats_bulk'])};", src)
                    assert n == 1, name
        open(p, "w").write(src)
        print("updated", p)


def apply_share(path: str, csrc: str = CSRC) -> None:
    """Result of `torchrun ... bench.py --gpus N --tune-share`: the thread split and the upsample share
    of the exchange pair, for two ranks (N <= 2) or for more (the `_wide` defaults)."""
    with open(path) as f:
        text = f.read()
    res = json.loads(text[text.index("{"):])
    suffix = "_wide" if int(res["n_gpus"]) > 2 else ""
    p = os.path.join(csrc, "dl_tuned.inc")
    src = open(p).read()
    if res["best"].get("pool"):       # the cursor form won: one thread split up to four ranks, one beyond
        wide = "_wide" if int(res["n_gpus"]) > 4 else ""
        pairs = (("kDefaultPool_upsample_bnstats_allreduce", 1),
                 (f"kDefaultPoolPair_upsample_bnstats_allreduce{wide}", res["best"]["index"]),
                 ("kBnStatsBulk_upsample_bnstats_allreduce", res["best"].get("bnstats_bulk", 0)))
    else:
        pairs = (("kDefaultPool_upsample_bnstats_allreduce", 0),
                 (f"kDefaultPair_upsample_bnstats_allreduce{suffix}", res["best"]["index"]),
                 (f"kDefaultShare_upsample_bnstats_allreduce{suffix}", res["best"]["share_permille"]),
                 ("kBnStatsBulk_upsample_bnstats_allreduce", res["best"].get("bnstats_bulk", 0)))
    for key, val in pairs:
        src, n = re.subn(rf"({key} = )\d+;", rf"\g<1>{int(val)};", src)
        assert n == 1, key
    open(p, "w").write(src)
    print("updated", p)


if __name__ == "__main__":
    if sys.argv[1] == "--share":
        apply_share(sys.argv[2])
    else:
        apply(sys.argv[1])
