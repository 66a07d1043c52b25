"""Launcher: the engine's OpenAI-compatible server on ``port + 1`` and the Dynasor proxy in
front of it on ``port`` (reference: arctic_inference/dynasor/vllm_server.py:49-107).

    python -m arcticinference_b200.dynasor.server MODEL --port 8000 [engine flags]
"""

from __future__ import annotations

import argparse
import signal
import subprocess
import sys
import time
import urllib.request


def wait_healthy(port: int, timeout: float = 1800.0, interval: float = 1.0, proc=None) -> bool:
    t0 = time.time()
    while time.time() - t0 < timeout:
        if proc is not None and proc.poll() is not None:
            return False
        try:
            with urllib.request.urlopen("http://127.0.0.1:%d/health" % port, timeout=2) as r:
                if r.status == 200:
                    return True
        except Exception:  # noqa: BLE001
            pass
        time.sleep(interval)
    return False


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description="engine server + Dynasor proxy", add_help=False)
    ap.add_argument("--port", type=int, default=8000)
    ap.add_argument("--host", default="0.0.0.0")
    ns, engine_args = ap.parse_known_args(argv)
    if "-h" in engine_args or "--help" in engine_args:
        print(__doc__)
        return 0
    engine_cmd = [sys.executable, "-m", "arcticinference_b200.cli", "serve", *engine_args,
                  "--host", "127.0.0.1", "--port", str(ns.port + 1)]
    engine = subprocess.Popen(engine_cmd)
    procs = [engine]

    def stop(*_):
        for p in procs:
            if p.poll() is None:
                p.terminate()

    signal.signal(signal.SIGINT, stop)
    signal.signal(signal.SIGTERM, stop)
    if not wait_healthy(ns.port + 1, proc=engine):
        stop()
        return 1
    proxy = subprocess.Popen([sys.executable, "-m", "arcticinference_b200.dynasor.openai_server",
                              "--host", ns.host, "--port", str(ns.port),
                              "--target", "http://127.0.0.1:%d" % (ns.port + 1)])
    procs.append(proxy)
    rc = engine.wait()
    stop()
    return rc


if __name__ == "__main__":
    sys.exit(main())
