"""Command line: ``python -m arcticinference_b200.cli <command>``.

    serve MODEL [engine flags] [--host H --port P]     OpenAI-compatible server
    server [--host H --port P]                          replica-pool REST server
    bench-embedding ...                                 see benchmarks/embedding_bench.py

``serve`` takes the flags the reference adds to ``vllm serve`` (README.md:98-124,
arctic_inference/vllm/args.py:33-69): ``--ulysses-sequence-parallel-size``,
``--enable-shift-parallel``, ``--shift-parallel-threshold``, ``--speculative-config``,
``--forest-cascade-attn-configs``, ``--fp32-lm-head``. A multi-GPU engine runs as one process
per GPU: ``serve`` started on its own with a parallel layout of N > 1 ranks launches those N
processes itself (``torch.distributed.run`` on this node, rendezvous on 127.0.0.1) and
becomes their parent, as the reference's ``vllm serve`` spawns its workers; started under
``torch.distributed.run`` (RANK set) it is one of the ranks. Rank 0 serves HTTP, the others
follow its requests.
"""

from __future__ import annotations

import argparse
import logging
import sys


def _free_port() -> int:
    """A rendezvous port below the kernel's ephemeral range (a port handed out by bind(0) can
    become the local end of another process's outgoing connection before rank 0 listens)."""
    import os
    import random
    import socket
    rng = random.Random(os.getpid() * 7919 + int.from_bytes(os.urandom(4), "little"))
    for _ in range(200):
        port = rng.randrange(15000, 30000)
        with socket.socket() as s:
            try:
                s.bind(("127.0.0.1", port))
            except OSError:
                continue
        return port
    raise RuntimeError("no free port for the ranks' rendezvous")


def rank_launch_command(argv: list, world: int, port: int) -> list:
    """The command that runs ``serve`` with ``argv`` as ``world`` ranks on this node."""
    return [sys.executable, "-m", "torch.distributed.run", "--nnodes=1",
            "--nproc-per-node", str(world), "--master-addr", "127.0.0.1",
            "--master-port", str(port), "-m", "arcticinference_b200.cli"] + list(argv)


def _spawn_ranks(argv: list, world: int) -> int:
    """Run the ranks as children and wait for them; an interrupt is passed on."""
    import signal
    import subprocess
    proc = subprocess.Popen(rank_launch_command(argv, world, _free_port()))
    for sig in (signal.SIGINT, signal.SIGTERM):
        signal.signal(sig, lambda s, _f: proc.send_signal(s))
    return proc.wait()


def _serve(ns: argparse.Namespace) -> int:
    import os
    from .config import EngineArgs
    from .engine.async_llm import AsyncLLM
    args = EngineArgs.from_cli_args(ns)
    world = (args.pipeline_parallel_size * args.tensor_parallel_size *
             args.ulysses_sequence_parallel_size)
    if world > 1 and "RANK" not in os.environ:
        return _spawn_ranks(ns.argv, world)
    llm = AsyncLLM.from_engine_args(args, device=ns.device)
    if not llm.is_leader:
        llm.run_follower()
        return 0
    import uvicorn
    from .entrypoints.openai_server import build_app
    llm.start()
    app = build_app(llm, args.served_model_name or args.model)
    try:
        uvicorn.run(app, host=ns.host, port=ns.port, log_level=ns.uvicorn_log_level)
    finally:
        llm.shutdown()
    return 0


def _server(ns: argparse.Namespace) -> int:
    import uvicorn
    from .server.api import app
    uvicorn.run(app, host=ns.host, port=ns.port, log_level="info")
    return 0


def make_parser() -> argparse.ArgumentParser:
    from .config import EngineArgs
    ap = argparse.ArgumentParser(prog="arcticinference_b200")
    sub = ap.add_subparsers(dest="command", required=True)
    s = sub.add_parser("serve", help="OpenAI-compatible server")
    s.add_argument("model", type=str)
    s.add_argument("--host", default="0.0.0.0")
    s.add_argument("--port", type=int, default=8000)
    s.add_argument("--device", default=None)
    s.add_argument("--uvicorn-log-level", default="info")
    # flags of `vllm serve` command lines that need nothing here: requests are not logged,
    # no checkpoint code is ever executed, statistics are served on /metrics only
    for flag in ("--disable-log-requests", "--trust-remote-code", "--disable-log-stats"):
        s.add_argument(flag, action="store_true", help="accepted for command-line compatibility")
    EngineArgs.add_cli_args(s)
    s.set_defaults(fn=_serve)
    r = sub.add_parser("server", help="replica-pool REST server (/init, /generate, ...)")
    r.add_argument("--host", default="0.0.0.0")
    r.add_argument("--port", type=int, default=8000)
    r.set_defaults(fn=_server)
    return ap


def main(argv=None) -> int:
    logging.basicConfig(level=logging.INFO)
    ns = make_parser().parse_args(argv)
    ns.argv = list(sys.argv[1:] if argv is None else argv)
    return ns.fn(ns)


if __name__ == "__main__":
    sys.exit(main())
