"""OpenAI-compatible ``/v1/embeddings`` front end for :class:`EmbeddingEngine`.

The reference compares its gRPC embedding service with an OpenAI HTTP endpoint
served by plain vLLM (benchmark/embedding/benchmark_http.py, run_benchmark.sh);
this module is that endpoint for this package's own engine, so both transports
can be measured against the same encoder.

Request body (``POST /v1/embeddings``): ``{"model": str, "input": str | [str] |
[int] | [[int]], "encoding_format": "float" | "base64", "dimensions": int?}``.
Response: ``{"object": "list", "data": [{"object": "embedding", "index": i,
"embedding": [...] | base64 of fp32 little-endian}], "model": ..., "usage":
{"prompt_tokens": n, "total_tokens": n}}``.

    python -m arcticinference_b200.embedding.http_server --model bert-base --port 8000
"""

from __future__ import annotations

import argparse
import base64
from typing import Optional

import numpy as np


def normalise_input(inp) -> list:
    """The four input shapes of the OpenAI schema -> list of prompts (str or token list)."""
    if isinstance(inp, str):
        return [inp]
    if not isinstance(inp, list) or not inp:
        raise ValueError("input must be a non-empty string or list")
    if all(isinstance(x, int) and not isinstance(x, bool) for x in inp):
        return [inp]
    if all(isinstance(x, str) for x in inp):
        return inp
    if all(isinstance(x, list) and x and all(isinstance(t, int) for t in x) for x in inp):
        return inp
    raise ValueError("input must be a string, a list of strings, a token list or a list of "
                     "token lists")


def build_app(async_engine, model_name: str = "embedding-model"):
    """FastAPI app over an :class:`AsyncEmbeddingEngine` (concurrent requests share batches)."""
    from fastapi import FastAPI, HTTPException
    from fastapi.responses import JSONResponse

    app = FastAPI(title="arcticinference_b200 embeddings")
    engine = async_engine.engine

    @app.get("/health")
    async def health():
        return {"status": "ok"}

    @app.get("/v1/models")
    async def models():
        return {"object": "list", "data": [{"id": model_name, "object": "model",
                                            "owned_by": "arcticinference_b200"}]}

    @app.get("/stats")
    async def stats():
        s = engine.stats
        return {k: getattr(s, k) for k in ("requests", "sequences", "tokens", "batches",
                                            "busy_seconds", "h2d_bytes", "d2h_bytes")}

    @app.post("/v1/embeddings")
    async def embeddings(body: dict):
        try:
            prompts = normalise_input(body.get("input"))
        except ValueError as e:
            raise HTTPException(status_code=400, detail=str(e))
        fmt = body.get("encoding_format", "float")
        if fmt not in ("float", "base64"):
            raise HTTPException(status_code=400, detail="encoding_format must be float or base64")
        dims: Optional[int] = body.get("dimensions")
        try:
            seqs = engine.tokenize(prompts)
            emb = await async_engine.encode(seqs)
        except ValueError as e:          # e.g. a sequence longer than the model allows
            raise HTTPException(status_code=400, detail=str(e))
        if dims is not None:
            if not 0 < int(dims) <= emb.shape[1]:
                raise HTTPException(status_code=400, detail="dimensions out of range")
            # shortened (Matryoshka-style) vectors are re-normalised
            emb = emb[:, :int(dims)]
            emb = emb / np.maximum(np.linalg.norm(emb, axis=1, keepdims=True), 1e-12)
        data = []
        for i, v in enumerate(emb):
            v = np.ascontiguousarray(v, dtype="<f4")
            data.append({"object": "embedding", "index": i,
                         "embedding": base64.b64encode(v.tobytes()).decode("ascii")
                         if fmt == "base64" else v.tolist()})
        n_tok = int(sum(len(s) for s in seqs))
        return JSONResponse({"object": "list", "data": data, "model": body.get("model", model_name),
                             "usage": {"prompt_tokens": n_tok, "total_tokens": n_tok}})

    return app


def main(argv=None) -> None:
    ap = argparse.ArgumentParser(description=__doc__,
                                 formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--model", default="bert-base")
    ap.add_argument("--host", default="0.0.0.0")
    ap.add_argument("--port", type=int, default=8000)
    ap.add_argument("--device", default=None)
    ap.add_argument("--pooling", default="cls", choices=["cls", "mean", "last"])
    ap.add_argument("--max-num-batched-tokens", type=int, default=16384)
    ap.add_argument("--max-wait-ms", type=float, default=1.0)
    a = ap.parse_args(argv)
    import uvicorn
    from .engine import AsyncEmbeddingEngine, EmbeddingEngine
    eng = EmbeddingEngine(a.model, device=a.device, pooling=a.pooling,
                          max_num_batched_tokens=a.max_num_batched_tokens)
    aeng = AsyncEmbeddingEngine(eng, max_wait_ms=a.max_wait_ms)
    try:
        uvicorn.run(build_app(aeng, a.model), host=a.host, port=a.port, log_level="warning")
    finally:
        aeng.stop()


if __name__ == "__main__":
    main()
