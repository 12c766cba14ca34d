"""Host-side pieces of ``bench.py`` that need no GPU."""

import json
import math
import subprocess
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))

import bench  # noqa: E402


def test_selfcheck_verdict_decides_between_ok_fallback_and_fail():
    good = {"loss_rel": 2e-5, "grad_rel": 4e-3, "param_rel_after_2_steps": 3e-3}
    assert bench.selfcheck_verdict(good, "auto") == ("ok", [])
    assert bench.selfcheck_verdict(good, "fused") == ("ok", [])
    bad = dict(good, grad_rel=0.08)
    assert bench.selfcheck_verdict(bad, "auto") == ("fallback", ["grad_rel"])
    assert bench.selfcheck_verdict(bad, "fused") == ("fail", ["grad_rel"])
    nan = dict(good, loss_rel=math.nan)
    assert bench.selfcheck_verdict(nan, "auto")[0] == "fallback"       # a NaN is never within the tolerance
    assert bench.selfcheck_verdict({"skipped": "peer-memory backend not active on this mesh"}, "auto") == ("ok", [])


def test_reference_arm_prints_one_unavailable_line_and_exits_zero():
    res = subprocess.run([sys.executable, str(ROOT / "bench.py"), "--impl", "reference", "--gpus", "1", "--steps", "2",
                          "--warmup", "1"], capture_output=True, text=True, timeout=300, cwd=str(ROOT))
    assert res.returncode == 0
    line = json.loads(res.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference" and "unavailable" in line
