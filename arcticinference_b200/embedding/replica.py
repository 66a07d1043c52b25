"""Embedding replica: a gRPC server in front of one :class:`EmbeddingEngine` (one GPU).

RPCs (``proto/inference.proto``): ``Encode`` (text prompts or pre-tokenised int32 byte
strings -> float32 byte strings), ``Abort``, ``GetReplicaInfo`` and ``HealthCheck``; same
behaviour as the reference's servicer (arctic_inference/embedding/replica.py:130-340),
including its error reporting through ``EncodeResponse.error`` rather than gRPC status codes.

    python -m arcticinference_b200.embedding.replica --model bert-base --port 50050
"""

from __future__ import annotations

import argparse
import asyncio
import logging
import signal
from typing import Optional

import grpc
import numpy as np

from . import messages as pb
from .engine import AsyncEmbeddingEngine, EmbeddingEngine

logger = logging.getLogger(__name__)

MAX_MESSAGE_BYTES = 1 << 30


class InferenceServicer:
    """The four RPC handlers. ``engine`` may be injected (tests use a CPU engine)."""

    def __init__(self, engine: EmbeddingEngine, model_name: Optional[str] = None):
        self.engine = engine
        self.async_engine = AsyncEmbeddingEngine(engine)
        self.model_name = model_name or engine.model_name
        self.ready = True

    def stop(self) -> None:
        self.ready = False
        self.async_engine.stop()

    # ---------------------------------------------------------------- RPCs
    async def Encode(self, request, context):
        rid = request.request_id
        resp = pb.EncodeResponse(request_id=rid)
        try:
            if request.model_name and request.model_name != self.model_name:
                raise ValueError("model %r is not served here (serving %r)" %
                                 (request.model_name, self.model_name))
            if len(request.token_id_bytes_i32) > 0:
                prompts = [np.frombuffer(b, dtype="<i4").tolist() for b in request.token_id_bytes_i32]
            else:
                prompts = list(request.prompts)
            if request.n_prompts and request.n_prompts != len(prompts):
                raise ValueError("n_prompts = %d but %d prompts were sent" %
                                 (request.n_prompts, len(prompts)))
            if not prompts:
                raise ValueError("no prompts")
            emb = await self.async_engine.encode(prompts, request_id=rid)
            resp.n_prompts = len(prompts)
            resp.embedding_dim = int(emb.shape[1])
            le = np.ascontiguousarray(emb, dtype="<f4")
            resp.embedding_bytes_fp32.extend(le[i].tobytes() for i in range(le.shape[0]))
        except Exception as e:  # noqa: BLE001 - reported in-band, like the reference
            logger.warning("Encode %s failed: %s", rid, e)
            resp.error = "%s: %s" % (type(e).__name__, e)
        return resp

    async def Abort(self, request, context):
        ok = self.async_engine.abort(request.request_id)
        return pb.AbortResponse(success=ok, message="" if ok else "request not pending")

    async def GetReplicaInfo(self, request, context):
        resp = pb.ReplicaInfoResponse(n_replicas=1, n_healthy_replicas=1 if self.ready else 0)
        e = self.engine
        resp.replica_infos.add(
            model_name=self.model_name, task="embed", dtype=str(e.encoder.dtype), ready=self.ready,
            parallel_config="one replica per GPU, device=%s" % e.device,
            decoding_config="pooling=%s normalize=%s" % (e.pooling, e.normalize),
            scheduler_config="max_num_batched_tokens=%d max_num_seqs=%d" % (e.max_tokens, e.max_seqs),
            lora_config="")
        return resp

    async def HealthCheck(self, request, context):
        return pb.HealthCheckResponse(healthy=self.ready, message="ok" if self.ready else "stopping")


def generic_handler(servicer) -> grpc.GenericRpcHandler:
    """gRPC method table for any object with the four coroutine methods."""
    table = {}
    for rpc in pb.METHODS:
        table[rpc] = grpc.unary_unary_rpc_method_handler(
            getattr(servicer, rpc),
            request_deserializer=pb.request_class(rpc).FromString,
            response_serializer=pb.response_class(rpc).SerializeToString)
    return grpc.method_handlers_generic_handler("%s.%s" % (pb.PACKAGE, pb.SERVICE), table)


class InferenceServer:
    def __init__(self, servicer, host: str = "0.0.0.0", port: int = 50050):
        self.servicer = servicer
        self.host, self.port = host, port
        self.server: Optional[grpc.aio.Server] = None

    async def start(self) -> int:
        self.server = grpc.aio.server(options=[
            ("grpc.max_send_message_length", MAX_MESSAGE_BYTES),
            ("grpc.max_receive_message_length", MAX_MESSAGE_BYTES)])
        self.server.add_generic_rpc_handlers((generic_handler(self.servicer),))
        self.port = self.server.add_insecure_port("%s:%d" % (self.host, self.port))
        await self.server.start()
        logger.info("embedding replica listening on %s:%d", self.host, self.port)
        return self.port

    async def stop(self, grace: float = 2.0) -> None:
        if self.server is not None:
            await self.server.stop(grace)
            self.server = None
        if hasattr(self.servicer, "stop"):
            self.servicer.stop()

    async def wait(self) -> None:
        await self.server.wait_for_termination()


def start_metrics_server(engine, port: int, host: str = "0.0.0.0"):
    """Serve the engine's counters in the Prometheus text format on ``port`` (its own registry;
    values are read from ``engine.stats`` at scrape time). Returns (server, thread)."""
    from prometheus_client import CollectorRegistry, start_http_server
    from prometheus_client.core import CounterMetricFamily, GaugeMetricFamily

    class Collector:
        def collect(self):
            st = engine.stats
            for name, doc in (("requests", "Encode requests served"),
                              ("sequences", "sequences embedded"), ("tokens", "tokens embedded"),
                              ("batches", "packed batches run"),
                              ("h2d_bytes", "bytes copied host to device"),
                              ("d2h_bytes", "bytes copied device to host")):
                c = CounterMetricFamily("ab200_embedding_" + name, doc)
                c.add_metric([], float(getattr(st, name)))
                yield c
            g = GaugeMetricFamily("ab200_embedding_busy_seconds", "seconds spent running batches")
            g.add_metric([], float(st.busy_seconds))
            yield g

    registry = CollectorRegistry()
    registry.register(Collector())
    return start_http_server(port, addr=host, registry=registry)


async def serve(args) -> None:
    engine = EmbeddingEngine(args.model, device=args.device,
                             max_num_batched_tokens=args.max_num_batched_tokens,
                             max_num_seqs=args.max_num_seqs, pooling=args.pooling)
    if getattr(args, "metrics_port", None):
        start_metrics_server(engine, args.metrics_port, args.host)
    server = InferenceServer(InferenceServicer(engine, args.served_model_name), args.host, args.port)
    await server.start()
    stop = asyncio.Event()
    loop = asyncio.get_running_loop()
    for sig in (signal.SIGINT, signal.SIGTERM):
        try:
            loop.add_signal_handler(sig, stop.set)
        except NotImplementedError:
            pass
    await stop.wait()
    await server.stop()


def make_parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(description="embedding replica (gRPC)")
    ap.add_argument("--model", default="bert-base")
    ap.add_argument("--served-model-name", default=None)
    ap.add_argument("--host", default="0.0.0.0")
    ap.add_argument("--port", type=int, default=50050)
    ap.add_argument("--device", default=None, help='e.g. "cuda:3"; default: cuda if present')
    ap.add_argument("--max-num-batched-tokens", type=int, default=16384)
    ap.add_argument("--max-num-seqs", type=int, default=2048)
    ap.add_argument("--pooling", default=None, choices=[None, "cls", "mean", "last"])
    ap.add_argument("--metrics-port", type=int, default=0,
                    help="serve Prometheus metrics on this port (0: off)")
    ap.add_argument("--workers", type=int, default=16, help="accepted for compatibility; the "
                    "server is asynchronous and needs no worker pool")
    return ap


if __name__ == "__main__":
    logging.basicConfig(level=logging.INFO)
    asyncio.run(serve(make_parser().parse_args()))
