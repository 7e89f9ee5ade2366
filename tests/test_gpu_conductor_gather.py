"""Live torch.compile(backend="gint") of the benchmark's conductor graph with the B200 executor installed and its conductor
fast path on: the row gather x[idx] that the conductor leaves to torch eager is folded into the fused program's launch
(two kernels of this library per call, no gather kernel), results equal torch eager; an index that cannot be folded
(int32) keeps torch's gather. Skipped where baseline/_ref is absent."""
import json
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

from baseline import ref_harness  # noqa: E402

pytestmark = [pytest.mark.gpu, pytest.mark.skipif(not ref_harness.available(), reason=ref_harness.why_unavailable() or "reference not installed")]


def test_conductor_graph_folds_its_gather():
    r = subprocess.run([sys.executable, os.path.join(ROOT, "tests", "conductor_gather_runner.py")], capture_output=True, text=True, timeout=900, cwd=ROOT)
    assert r.returncode == 0, r.stderr[-4000:]
    res = json.loads(r.stdout.strip().splitlines()[-1])
    for name in ("positive", "negative"):
        c = res[name]
        assert c["foldable"] == 1 and c["folded"] >= 2, c              # folded on both calls
        assert c["launches_per_call"] == 2, c                            # fused program + row sum; the gather kernel is gone
        assert c["z_close"] and c["s_close"], c
    assert res["programs_equal_recorded"], res["live_program_lengths"]    # the live conductor emits the recorded 155- and 24-instruction streams
    c = res["int32"]
    assert c["folded"] == 0 and c["launches_per_call"] == 2 and c["z_close"] and c["s_close"], c
