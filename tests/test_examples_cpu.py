"""The offline examples run end to end (tiny built-in architectures, CPU)."""

import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.parametrize("script,model,expect", [
    ("ulysses.py", "llama-tiny", "800 generated"),
    ("swiftkv.py", "llama-tiny-swiftkv", "800 generated"),
    ("spec_decode.py", "llama-tiny", "drafted per position: ["),
])
def test_offline_example(script, model, expect):
    env = dict(os.environ, OMP_NUM_THREADS="1", CUDA_VISIBLE_DEVICES="")
    for k in ("RANK", "WORLD_SIZE", "LOCAL_RANK"):
        env.pop(k, None)
    p = subprocess.run([sys.executable, os.path.join(ROOT, "examples", "offline", script), model],
                       capture_output=True, text=True, timeout=600, env=env)
    assert p.returncode == 0, p.stderr[-2000:]
    assert expect in p.stdout and "145 prompt tokens" in p.stdout
