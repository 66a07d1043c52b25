"""``python -m arcticinference_b200.server.cli [--host H] [--port P] [--multi-model]``:
start the replica-pool REST server (reference: arctic_inference/server/cli.py:1-30)."""

from __future__ import annotations

import argparse


def main(argv=None) -> None:
    ap = argparse.ArgumentParser(description="replica-pool REST server")
    ap.add_argument("--host", default="0.0.0.0")
    ap.add_argument("--port", type=int, default=8000)
    ap.add_argument("--multi-model", action="store_true",
                    help="serve several models, GPUs shared evenly between them")
    ap.add_argument("--log-level", default="info")
    ns = ap.parse_args(argv)
    import uvicorn
    from . import api
    if ns.multi_model:
        api.use_driver()
    uvicorn.run(api.app, host=ns.host, port=ns.port, log_level=ns.log_level)


if __name__ == "__main__":
    main()
