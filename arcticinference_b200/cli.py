"""Command line: ``python -m arcticinference_b200.cli <command>``.

    serve MODEL [engine flags] [--host H --port P]     OpenAI-compatible server
    server [--host H --port P]                          replica-pool REST server
    bench-embedding ...                                 see benchmarks/embedding_bench.py

``serve`` takes the flags the reference adds to ``vllm serve`` (README.md:98-124,
arctic_inference/vllm/args.py:33-69): ``--ulysses-sequence-parallel-size``,
``--enable-shift-parallel``, ``--shift-parallel-threshold``, ``--speculative-config``,
``--forest-cascade-attn-configs``, ``--fp32-lm-head``. A multi-GPU engine is started as one
process per GPU (``python -m torch.distributed.run --nproc-per-node N -m
arcticinference_b200.cli serve ...``); rank 0 serves HTTP, the others follow its requests.
"""

from __future__ import annotations

import argparse
import logging
import sys


def _serve(ns: argparse.Namespace) -> int:
    from .config import EngineArgs
    from .engine.async_llm import AsyncLLM
    args = EngineArgs.from_cli_args(ns)
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
    return ns.fn(ns)


if __name__ == "__main__":
    sys.exit(main())
