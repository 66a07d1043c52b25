"""Asynchronous client of the embedding service (a replica or a replica manager).

    async with InferenceClient("127.0.0.1", 60050) as c:
        vectors = await c.embed(["some text", "more text"])          # np.ndarray [2, dim]
        vectors = await c.embed(token_ids=[[101, 2023, 102], [101, 102]])

Mirrors the calls of the reference client (arctic_inference/embedding/client.py:69-256).
"""

from __future__ import annotations

import uuid
from typing import Optional, Sequence

import grpc
import numpy as np

from . import messages as pb

MAX_MESSAGE_BYTES = 1 << 30


class EmbeddingError(RuntimeError):
    pass


class InferenceClient:
    def __init__(self, host: str = "127.0.0.1", port: int = 50050, timeout: Optional[float] = 60.0):
        self.target = "%s:%d" % (host, port)
        self.timeout = timeout
        self.channel: Optional[grpc.aio.Channel] = None
        self._calls: dict = {}

    async def connect(self) -> None:
        self.channel = grpc.aio.insecure_channel(self.target, options=[
            ("grpc.max_send_message_length", MAX_MESSAGE_BYTES),
            ("grpc.max_receive_message_length", MAX_MESSAGE_BYTES)])
        for rpc in pb.METHODS:
            self._calls[rpc] = self.channel.unary_unary(
                pb.method_path(rpc),
                request_serializer=pb.request_class(rpc).SerializeToString,
                response_deserializer=pb.response_class(rpc).FromString)

    async def close(self) -> None:
        if self.channel is not None:
            await self.channel.close()
            self.channel = None

    async def __aenter__(self):
        await self.connect()
        return self

    async def __aexit__(self, *exc):
        await self.close()

    async def _call(self, rpc: str, request):
        if self.channel is None:
            await self.connect()
        return await self._calls[rpc](request, timeout=self.timeout)

    # ------------------------------------------------------------------ calls
    async def embed(self, prompts: Optional[Sequence[str]] = None,
                    token_ids: Optional[Sequence[Sequence[int]]] = None, model_name: str = "",
                    request_id: Optional[str] = None, priority: int = 0) -> np.ndarray:
        if (prompts is None) == (token_ids is None):
            raise ValueError("pass either prompts or token_ids")
        req = pb.EncodeRequest(request_id=request_id or uuid.uuid4().hex, model_name=model_name,
                               priority=priority)
        if prompts is not None:
            req.prompts.extend(prompts)
            req.n_prompts = len(prompts)
        else:
            req.token_id_bytes_i32.extend(np.asarray(t, dtype="<i4").tobytes() for t in token_ids)
            req.n_prompts = len(token_ids)
        resp = await self._call("Encode", req)
        if resp.error:
            raise EmbeddingError(resp.error)
        dim = resp.embedding_dim
        out = np.empty((resp.n_prompts, dim), dtype=np.float32)
        for i, b in enumerate(resp.embedding_bytes_fp32):
            out[i] = np.frombuffer(b, dtype="<f4", count=dim)
        return out

    async def abort(self, request_id: str) -> dict:
        r = await self._call("Abort", pb.AbortRequest(request_id=request_id))
        return {"success": r.success, "message": r.message}

    async def get_replica_info(self) -> dict:
        r = await self._call("GetReplicaInfo", pb.ReplicaInfoRequest())
        return {"n_replicas": r.n_replicas, "n_healthy_replicas": r.n_healthy_replicas,
                "message": r.message,
                "replicas": [{f.name: getattr(i, f.name) for f in i.DESCRIPTOR.fields}
                             for i in r.replica_infos]}

    async def health_check(self) -> bool:
        try:
            r = await self._call("HealthCheck", pb.HealthCheckRequest())
            return bool(r.healthy)
        except grpc.aio.AioRpcError:
            return False
