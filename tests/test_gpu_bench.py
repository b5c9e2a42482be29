"""bench.py's side modes on a GPU box: the speedup-vs-ratio study and the single-item runs that
the profiles are taken from must run and produce sane rows (their numbers are not asserted)."""
import json
import os
import subprocess
import sys

import pytest

from conftest import ROOT

pytestmark = pytest.mark.gpu


def _bench(*flags):
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), *flags], capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    return [json.loads(line) for line in r.stdout.splitlines() if line.startswith("{")]


def test_speedup_vs_ratio_study_short_form(dev):
    (out,) = _bench("--study", "--quick")
    rows = out["study"]
    assert len(rows) == 6
    for row in rows:
        assert row["pair"] in ("upsample_bnstats", "histc_maxpool")
        assert row["first_us"] > 0 and row["second_us"] > 0 and row["back_to_back_us"] > 0
        # the fused pair can neither be much slower than back to back nor faster than its slower half
        assert 0.6 < row["speedup_horizontal"] < 2.0
        assert row["horizontal_us"] >= 0.9 * max(row["first_us"], row["second_us"]) - 3.0
    # the halves' ratio moves with the scale of the second half
    ratios = [r["ratio_first_over_second"] for r in rows if r["pair"] == "histc_maxpool"]
    assert ratios[0] > ratios[1] > ratios[2]


def test_single_items_for_profiling(dev):
    out = _bench("--only", "cfg1:a,cfg1:b,cfg1:fused,maxpool_bnstats:fused,blake256_sia:fused", "--steps", "2", "--warmup", "1",
                 "--count", "1048576")
    assert [o["only"] for o in out] == ["upsample_bnstats", "upsample_bnstats", "upsample_bnstats", "maxpool_bnstats", "blake256_sia"]
    assert all((o.get("us_per_step") or o.get("ms_per_step")) > 0 for o in out)
