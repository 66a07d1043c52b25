"""The benchmark's reference arm must answer on any machine: one JSON line, exit code 0."""

import json
import os
import subprocess
import sys

REPO = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_reference_arm_reports_unavailable():
    p = subprocess.run([sys.executable, os.path.join(REPO, "bench.py"), "--impl", "reference", "--gpus", "1",
                        "--steps", "1", "--warmup", "3"], capture_output=True, text=True, timeout=300)
    assert p.returncode == 0, p.stderr[-500:]
    line = [l for l in p.stdout.splitlines() if l.startswith("{")][-1]
    d = json.loads(line)
    assert d["impl"] == "reference" and isinstance(d["unavailable"], str) and d["unavailable"]
