"""``serve`` with a multi-rank layout starts its own ranks (the reference's ``vllm serve``
spawns its workers: README.md:98-124)."""

import json
import os
import signal
import subprocess
import sys
import time
import urllib.request

import pytest

from arcticinference_b200 import cli
from tests._mp_util import free_port

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_rank_launch_command_names_every_rank_and_loopback():
    cmd = cli.rank_launch_command(["serve", "m", "--tensor-parallel-size", "4"], 4, 12345)
    assert cmd[0] == sys.executable and "torch.distributed.run" in cmd
    assert cmd[cmd.index("--nproc-per-node") + 1] == "4"
    assert cmd[cmd.index("--master-addr") + 1] == "127.0.0.1"
    assert cmd[cmd.index("--master-port") + 1] == "12345"
    assert cmd[-4:] == ["serve", "m", "--tensor-parallel-size", "4"]


def test_serve_spawns_ranks_only_when_started_alone(monkeypatch):
    seen = {}
    monkeypatch.setattr(cli, "_spawn_ranks", lambda argv, world: seen.update(argv=argv, world=world) or 0)
    monkeypatch.delenv("RANK", raising=False)
    argv = ["serve", "llama-tiny", "--device", "cpu", "--tensor-parallel-size", "2"]
    assert cli.main(argv) == 0
    assert seen == {"argv": argv, "world": 2}


@pytest.mark.timeout(240)
def test_two_rank_serve_answers_a_completion_on_cpu():
    port = free_port()
    env = dict(os.environ, PYTHONPATH=ROOT, ARCTIC_B200_NO_AUTOBUILD="1")
    env.pop("RANK", None)
    proc = subprocess.Popen(
        [sys.executable, "-m", "arcticinference_b200.cli", "serve", "llama-tiny", "--device", "cpu",
         "--tensor-parallel-size", "2", "--comm-backend", "nccl", "--host", "127.0.0.1",
         "--port", str(port), "--max-model-len", "128", "--uvicorn-log-level", "warning"],
        cwd=ROOT, env=env, start_new_session=True)
    try:
        base = "http://127.0.0.1:%d" % port
        deadline = time.time() + 180
        while True:
            assert proc.poll() is None, "serve exited with %s" % proc.returncode
            try:
                with urllib.request.urlopen(base + "/health", timeout=2) as r:
                    if r.status == 200:
                        break
            except OSError:
                pass
            assert time.time() < deadline, "server did not come up"
            time.sleep(1.0)
        body = json.dumps({"model": "llama-tiny", "prompt": [5, 6, 7, 8], "max_tokens": 4,
                           "temperature": 0}).encode()
        req = urllib.request.Request(base + "/v1/completions", data=body,
                                     headers={"Content-Type": "application/json"})
        with urllib.request.urlopen(req, timeout=60) as r:
            out = json.loads(r.read())
        assert out["usage"]["completion_tokens"] == 4
    finally:
        os.killpg(proc.pid, signal.SIGTERM)
        try:
            proc.wait(timeout=30)
        except subprocess.TimeoutExpired:
            os.killpg(proc.pid, signal.SIGKILL)
            proc.wait(timeout=10)
