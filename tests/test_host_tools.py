"""Host-side tools that need no GPU: writing a sweep result into the compiled defaults, and the
benchmark's CPU arm (the oracle port timed on the host cores)."""
import json
import os
import re
import shutil
import subprocess
import sys

from conftest import ROOT
from hfuse_b200 import apply_tuning


def _value(text, name):
    return int(re.search(rf"{name} = (-?\d+);", text).group(1))


def test_sweep_results_are_written_into_the_default_tables(tmp_path):
    csrc = tmp_path / "csrc"
    csrc.mkdir()
    for inc in ("dl_tuned.inc", "crypto_tuned.inc"):
        shutil.copy(os.path.join(apply_tuning.CSRC, inc), csrc / inc)
    before = (csrc / "crypto_tuned.inc").read_text()
    sweep = {"solo": {"histc": {"best": 4, "variant": "512:0:4", "us": 1.0},
                      "im2col": {"best": 1, "variant": "256:0:8", "us": 1.0, "im2col_bulk": 0}},
             "pair": {"im2col_histc": {"best": 3, "variant": "256:256:3", "us": 1.0, "im2col_bulk": 1, "histc_bulk": 1},
                      "histc_bnstats": {"best": 9, "variant": "512:256:1", "us": 1.0, "bnstats_bulk": 1, "histc_bulk": 0}}}
    path = tmp_path / "tune.json"
    path.write_text("some log line\n" + json.dumps(sweep))          # text ahead of the JSON is skipped
    apply_tuning.apply(str(path), str(csrc))
    dl = (csrc / "dl_tuned.inc").read_text()
    assert _value(dl, "kDefaultSolo_histc") == 4 and _value(dl, "kDefaultSolo_im2col") == 1
    assert _value(dl, "kDefaultPair_im2col_histc") == 3 and _value(dl, "kDefaultPair_histc_bnstats") == 9
    assert _value(dl, "kIm2colBulk_im2col") == 0 and _value(dl, "kIm2colBulk_im2col_histc") == 1
    assert _value(dl, "kHistcBulk_im2col_histc") == 1 and _value(dl, "kHistcBulk_histc_bnstats") == 0
    assert _value(dl, "kBnStatsBulk_histc_bnstats") == 1
    assert (csrc / "crypto_tuned.inc").read_text() == before          # nothing in the sweep for it
    share = {"pair": "upsample_bnstats_allreduce", "n_gpus": 8, "best": {"index": 16, "share_permille": 300}}
    path.write_text(json.dumps(share))
    apply_tuning.apply_share(str(path), str(csrc))
    dl = (csrc / "dl_tuned.inc").read_text()
    assert _value(dl, "kDefaultPair_upsample_bnstats_allreduce_wide") == 16
    assert _value(dl, "kDefaultShare_upsample_bnstats_allreduce_wide") == 300
    share["best"] = {"index": 16, "share_permille": -1, "pool": True, "bnstats_bulk": 1}       # cursor form, eight ranks
    path.write_text(json.dumps(share))
    apply_tuning.apply_share(str(path), str(csrc))
    dl = (csrc / "dl_tuned.inc").read_text()
    assert _value(dl, "kDefaultPool_upsample_bnstats_allreduce") == 1
    assert _value(dl, "kDefaultPoolPair_upsample_bnstats_allreduce_wide") == 16
    assert _value(dl, "kBnStatsBulk_upsample_bnstats_allreduce") == 1
    share["n_gpus"], share["best"] = 4, {"index": 7, "share_permille": -1, "pool": True}          # up to four ranks
    path.write_text(json.dumps(share))
    apply_tuning.apply_share(str(path), str(csrc))
    dl = (csrc / "dl_tuned.inc").read_text()
    assert _value(dl, "kDefaultPoolPair_upsample_bnstats_allreduce") == 7
    assert _value(dl, "kDefaultPoolPair_upsample_bnstats_allreduce_wide") == 16
    assert _value(dl, "kBnStatsBulk_upsample_bnstats_allreduce") == 0
    share["n_gpus"], share["best"] = 2, {"index": 20, "share_permille": 100}
    path.write_text(json.dumps(share))
    apply_tuning.apply_share(str(path), str(csrc))
    dl = (csrc / "dl_tuned.inc").read_text()
    assert _value(dl, "kDefaultPair_upsample_bnstats_allreduce") == 20
    assert _value(dl, "kDefaultShare_upsample_bnstats_allreduce") == 100


def test_reference_arm_of_the_benchmark_runs_on_the_host():
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--steps", "2", "--warmup", "1"],
                       capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stderr[-2000:]
    line = json.loads(r.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference" and line["steps"] == 2 and line["warmup"] == 1
    assert line["unit"] == "GB/s" and line["value"] > 0 and line["higher_is_better"] is True
    assert line["cpu_baseline"]["kind"] == "port" and line["cpu_baseline"]["cores"] >= 1
    assert line["e2e"]["value"] == line["value"] and line["e2e"]["h2d_bytes_per_step"] == 0
    assert "config 1" in line["config"]["workload"]
