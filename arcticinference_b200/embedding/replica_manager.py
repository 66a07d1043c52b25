"""Replica manager: launches embedding replicas, watches their health and balances requests.

The reference starts its N replicas on the *same* GPU to fill it with small batches
(arctic_inference/embedding/replica_manager.py:138-158,243-289). A B200 is filled by one
engine with a 16k-token packed batch, so the default here is one replica per visible GPU
(``--gpus-per-node`` / ``--devices``); ``--replicas-per-gpu`` restores the stacked layout.
Load balancing (round_robin, least_loaded, random), the health loop that takes a replica out
of rotation and puts it back, and the forwarding gRPC front end follow the reference
(:173-199, :305-346, :354-407).

    python -m arcticinference_b200.embedding.replica_manager --model bert-base --num-replicas 8
"""

from __future__ import annotations

import argparse
import asyncio
import logging
import os
import random
import signal
import socket
import subprocess
import sys
from dataclasses import dataclass
from enum import Enum
from typing import Optional

import grpc

from . import messages as pb
from .client import InferenceClient
from .replica import InferenceServer

logger = logging.getLogger(__name__)


class LoadBalancing(str, Enum):
    ROUND_ROBIN = "round_robin"
    LEAST_LOADED = "least_loaded"
    RANDOM = "random"


@dataclass
class ReplicaInfo:
    host: str
    port: int
    device: Optional[str] = None
    process: Optional[subprocess.Popen] = None
    client: Optional[InferenceClient] = None
    healthy: bool = False
    inflight: int = 0
    served: int = 0
    failures: int = 0

    async def close(self) -> None:
        if self.client is not None:
            await self.client.close()
            self.client = None
        if self.process is not None and self.process.poll() is None:
            self.process.terminate()
            try:
                self.process.wait(timeout=10)
            except subprocess.TimeoutExpired:
                self.process.kill()


def port_is_free(host: str, port: int) -> bool:
    with socket.socket(socket.AF_INET, socket.SOCK_STREAM) as s:
        s.setsockopt(socket.SOL_SOCKET, socket.SO_REUSEADDR, 1)
        try:
            s.bind((host if host != "0.0.0.0" else "", port))
            return True
        except OSError:
            return False


class ReplicaManager:
    def __init__(self, replicas: Optional[list] = None, load_balancing: str = "round_robin",
                 health_interval: float = 2.0, forward_timeout: float = 20.0,
                 startup_timeout: float = 60.0):
        self.replicas: list = list(replicas or [])
        self.policy = LoadBalancing(load_balancing)
        self.health_interval = health_interval
        self.forward_timeout = forward_timeout
        self.startup_timeout = startup_timeout
        self._rr = 0
        self._health_task: Optional[asyncio.Task] = None
        self._rng = random.Random(0)

    # ---------------------------------------------------------------- lifecycle
    def build_replica_cmd(self, model: str, host: str, port: int, device: Optional[str],
                          extra: Optional[list] = None) -> list:
        cmd = [sys.executable, "-m", "arcticinference_b200.embedding.replica", "--model", model,
               "--host", host, "--port", str(port)]
        if device:
            cmd += ["--device", device]
        return cmd + list(extra or [])

    async def launch(self, model: str, num_replicas: int, base_port: int, host: str = "127.0.0.1",
                     devices: Optional[list] = None, extra: Optional[list] = None) -> None:
        """Start ``num_replicas`` replica processes on ports base_port+1.. and wait until all
        answer their health check."""
        port = base_port
        for i in range(num_replicas):
            port += 1
            while not port_is_free(host, port):
                port += 1
            dev = devices[i % len(devices)] if devices else None
            cmd = self.build_replica_cmd(model, host, port, dev, extra)
            logger.info("starting replica %d: %s", i, " ".join(cmd))
            proc = subprocess.Popen(cmd, env=dict(os.environ))
            self.replicas.append(ReplicaInfo(host, port, dev, proc))
        await self.start()
        deadline = asyncio.get_running_loop().time() + self.startup_timeout
        while asyncio.get_running_loop().time() < deadline:
            await self.check_all()
            if all(r.healthy for r in self.replicas):
                return
            dead = [r for r in self.replicas if r.process is not None and r.process.poll() is not None]
            if dead:
                raise RuntimeError("replica on port %d exited with code %s during start-up" %
                                   (dead[0].port, dead[0].process.returncode))
            await asyncio.sleep(0.5)
        raise TimeoutError("replicas not healthy after %.0f s" % self.startup_timeout)

    async def start(self) -> None:
        for r in self.replicas:
            if r.client is None:
                r.client = InferenceClient(r.host, r.port, timeout=self.forward_timeout)
                await r.client.connect()
        await self.check_all()
        if self._health_task is None:
            self._health_task = asyncio.create_task(self._health_loop())

    async def stop(self) -> None:
        if self._health_task is not None:
            self._health_task.cancel()
            try:
                await self._health_task
            except (asyncio.CancelledError, Exception):  # noqa: BLE001
                pass
            self._health_task = None
        for r in self.replicas:
            await r.close()

    # ---------------------------------------------------------------- health
    async def check_all(self) -> None:
        res = await asyncio.gather(*[r.client.health_check() for r in self.replicas],
                                   return_exceptions=True)
        for r, ok in zip(self.replicas, res):
            now = ok is True
            if now != r.healthy:
                logger.info("replica %s:%d is now %s", r.host, r.port, "healthy" if now else "unhealthy")
            r.healthy = now

    async def _health_loop(self) -> None:
        while True:
            await asyncio.sleep(self.health_interval)
            try:
                await self.check_all()
            except Exception as e:  # noqa: BLE001
                logger.warning("health check round failed: %s", e)

    # ---------------------------------------------------------------- routing
    def select_replica(self) -> Optional[ReplicaInfo]:
        live = [r for r in self.replicas if r.healthy]
        if not live:
            return None
        if self.policy is LoadBalancing.ROUND_ROBIN:
            self._rr = (self._rr + 1) % len(live)
            return live[self._rr]
        if self.policy is LoadBalancing.LEAST_LOADED:
            return min(live, key=lambda r: (r.inflight, r.served))
        return self._rng.choice(live)

    async def route(self, rpc: str, request):
        """Forward one request; a transport failure marks the replica unhealthy and the request
        is retried once on another replica."""
        last_err = None
        for _ in range(2):
            r = self.select_replica()
            if r is None:
                break
            r.inflight += 1
            try:
                resp = await r.client._call(rpc, request)
                r.served += 1
                return resp
            except grpc.aio.AioRpcError as e:
                r.failures += 1
                r.healthy = False
                last_err = e
            finally:
                r.inflight -= 1
        resp = pb.response_class(rpc)()
        msg = "no healthy replica" if last_err is None else "replica failed: %s" % last_err.details()
        if rpc == "Encode":
            resp.request_id = request.request_id
            resp.error = msg
        elif hasattr(resp, "message"):
            resp.message = msg
        return resp


class ManagerServicer:
    """gRPC front end: Encode is routed to one replica, Abort is broadcast, info and health are
    aggregated."""

    def __init__(self, manager: ReplicaManager):
        self.manager = manager

    async def Encode(self, request, context):
        return await self.manager.route("Encode", request)

    async def Abort(self, request, context):
        res = await asyncio.gather(*[r.client._call("Abort", request) for r in self.manager.replicas
                                     if r.healthy], return_exceptions=True)
        ok = any(getattr(x, "success", False) for x in res)
        return pb.AbortResponse(success=ok, message="" if ok else "request not pending on any replica")

    async def GetReplicaInfo(self, request, context):
        out = pb.ReplicaInfoResponse(n_replicas=len(self.manager.replicas),
                                     n_healthy_replicas=sum(r.healthy for r in self.manager.replicas))
        res = await asyncio.gather(*[r.client._call("GetReplicaInfo", request)
                                     for r in self.manager.replicas if r.healthy],
                                   return_exceptions=True)
        for x in res:
            if isinstance(x, Exception):
                out.message = "some replicas did not answer"
                continue
            for info in x.replica_infos:
                out.replica_infos.add().CopyFrom(info)
        return out

    async def HealthCheck(self, request, context):
        n = sum(r.healthy for r in self.manager.replicas)
        return pb.HealthCheckResponse(healthy=n > 0, message="%d/%d replicas healthy" %
                                      (n, len(self.manager.replicas)))


async def serve(args) -> None:
    mgr = ReplicaManager(load_balancing=args.load_balancing, health_interval=args.health_interval,
                         forward_timeout=args.forward_timeout, startup_timeout=args.startup_timeout)
    devices = args.devices.split(",") if args.devices else None
    if devices is None:
        try:
            import torch
            n = torch.cuda.device_count()
        except Exception:  # noqa: BLE001
            n = 0
        if n:
            devices = ["cuda:%d" % (i // args.replicas_per_gpu % n)
                       for i in range(args.num_replicas)] if args.replicas_per_gpu > 1 else \
                ["cuda:%d" % (i % n) for i in range(args.num_replicas)]
    extra = ["--max-num-batched-tokens", str(args.max_num_batched_tokens)]
    await mgr.launch(args.model, args.num_replicas, args.port, "127.0.0.1", devices, extra)
    server = InferenceServer(ManagerServicer(mgr), args.host, args.port)
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
    await mgr.stop()


def make_parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(description="embedding replica manager (gRPC)")
    ap.add_argument("--model", default="bert-base")
    ap.add_argument("--host", default="0.0.0.0")
    ap.add_argument("--port", type=int, default=60050)
    ap.add_argument("--num-replicas", type=int, default=2)
    ap.add_argument("--replicas-per-gpu", type=int, default=1)
    ap.add_argument("--devices", default=None, help='comma list, e.g. "cuda:0,cuda:1"')
    ap.add_argument("--load-balancing", default="round_robin",
                    choices=[e.value for e in LoadBalancing])
    ap.add_argument("--health-interval", type=float, default=2.0)
    ap.add_argument("--forward-timeout", type=float, default=20.0)
    ap.add_argument("--startup-timeout", type=float, default=60.0)
    ap.add_argument("--max-num-batched-tokens", type=int, default=16384)
    ap.add_argument("--workers", type=int, default=16, help="accepted for compatibility")
    return ap


def main_cli(argv=None) -> None:
    logging.basicConfig(level=logging.INFO)
    asyncio.run(serve(make_parser().parse_args(argv)))


if __name__ == "__main__":
    main_cli()
