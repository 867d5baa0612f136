"""The microbenchmark behind the rule that MMA and producer warps issue from an elected lane runs, and shows it."""
import re
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu


def test_issue_bench_runs_and_the_elected_lane_is_cheaper():
    proc = subprocess.run([sys.executable, "-m", "qorvix_b200.issue_bench"], capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stdout + proc.stderr
    figures = {}
    for line in proc.stdout.splitlines():
        m = re.match(r"(.+?)\s+(\d+) clocks a batch", line)
        if m:
            figures[m.group(1).strip()] = int(m.group(2))
    assert len(figures) == 9, proc.stdout
    elected = figures["elected lane, SS and TS in turn, two satisfied waits a batch"]
    lane0 = figures["lane-0 branch, SS and TS in turn, two satisfied waits a batch"]
    # eight products of 64 clocks each are the floor; the lane-0 form measured ~1,000 clocks, the elected lane ~600
    assert 500 <= elected < lane0, proc.stdout
