"""Data-parallel serving front: ``b200-serve serve MODEL --data-parallel-size N`` starts N engine servers (one per
GPU, or per ``--tensor-parallel-size`` group is NOT done here: replicas are single-GPU processes) on private ports and
one HTTP front on the public port that spreads the requests over them.

* Balancing: least outstanding requests, ties to the replica that has served fewest; a request may pin a replica with the
  ``X-data-parallel-rank`` header (upstream's external-balancing hook).
* Streaming answers are relayed chunk by chunk; everything else is relayed whole.
* A replica that stops answering is taken out of rotation (its in-flight requests fail with 502) and is probed again
  every few seconds; ``/health`` reports 200 while at least one replica serves.
* ``/metrics`` concatenates the replicas' Prometheus text with a ``replica="i"`` label; ``/scale_elastic_ep``
  (``{"new_data_parallel_size": n}``) starts or retires replica processes between requests.

The relay is a plain ASGI application over ``httpx``; replicas are addressed through a client factory so that tests can
mount in-process applications instead of sockets.
Parity: ``vllm serve --data-parallel-size`` with internal load balancing, which the reference's deployments use
(tests/v1/test_internal_lb_dp.py in its tree), and the scaling request of examples/ray_serving/elastic_ep/scale.py.
"""
# (no postponed annotations: the web framework resolves the handlers' parameter annotations at decoration time)
import asyncio
import json
import os
import subprocess
import sys
import time
from typing import Callable, Optional


class Replica:
    def __init__(self, rank: int, base_url: str, client, proc: Optional[subprocess.Popen] = None) -> None:
        self.rank, self.base_url, self.client, self.proc = rank, base_url, client, proc
        self.outstanding = 0
        self.healthy = True
        self.served = 0
        self.last_probe = 0.0


class DataParallelFront:
    """``clients``: one ``httpx.AsyncClient`` per replica (base URL set).  ``spawn(rank) -> Replica`` / ``retire(replica)``
    are only needed for elastic scaling."""

    PROBE_EVERY_S = 3.0

    def __init__(self, replicas: list, spawn: Optional[Callable] = None, retire: Optional[Callable] = None):
        self.replicas = list(replicas)
        self.spawn, self.retire = spawn, retire
        self._lock = asyncio.Lock()

    # ------------------------------------------------------------------ balancing
    def pick(self, pinned: Optional[int] = None) -> Optional[Replica]:
        if pinned is not None:
            if not 0 <= pinned < len(self.replicas):
                raise ValueError(f"data-parallel rank {pinned} outside [0, {len(self.replicas)})")
            return self.replicas[pinned]
        live = [r for r in self.replicas if r.healthy]
        return min(live, key=lambda r: (r.outstanding, r.served, r.rank)) if live else None

    async def probe(self, r: Replica) -> bool:
        r.last_probe = time.monotonic()
        try:
            resp = await r.client.get("/health", timeout=2.0)
            r.healthy = resp.status_code == 200
        except Exception:  # noqa: BLE001
            r.healthy = False
        return r.healthy

    async def revive(self) -> None:
        now = time.monotonic()
        for r in self.replicas:
            if not r.healthy and now - r.last_probe > self.PROBE_EVERY_S:
                await self.probe(r)

    # ------------------------------------------------------------------ application
    def build_app(self):
        from fastapi import FastAPI, Request
        from fastapi.responses import JSONResponse, PlainTextResponse, Response, StreamingResponse

        app = FastAPI(title="vllm_metax_b200 data-parallel front")
        front = self

        def err(code: int, msg: str):
            return JSONResponse({"error": {"message": msg, "type": "dp_front", "code": code}}, status_code=code)

        @app.get("/health")
        async def health():
            await front.revive()
            live = sum(r.healthy for r in front.replicas)
            return JSONResponse({"replicas": len(front.replicas), "healthy": live}, status_code=200 if live else 503)

        @app.get("/metrics")
        async def metrics():
            parts = []
            for r in front.replicas:
                try:
                    text = (await r.client.get("/metrics", timeout=5.0)).text
                except Exception:  # noqa: BLE001
                    continue
                for line in text.splitlines():
                    if line.startswith("#") or not line.strip():
                        parts.append(line)
                        continue
                    name, _, value = line.rpartition(" ")
                    name = (name[:-1] + f',replica="{r.rank}"}}') if name.endswith("}") else name + f'{{replica="{r.rank}"}}'
                    parts.append(f"{name} {value}")
            parts.append(f"b200:dp_front_replicas {len(front.replicas)}")
            for r in front.replicas:
                parts.append(f'b200:dp_front_requests_total{{replica="{r.rank}"}} {r.served}')
                parts.append(f'b200:dp_front_outstanding{{replica="{r.rank}"}} {r.outstanding}')
            return PlainTextResponse("\n".join(parts) + "\n")

        @app.post("/scale_elastic_ep")
        async def scale(req: Request):
            body = await req.json()
            n = int(body.get("new_data_parallel_size", 0))
            if n < 1:
                return err(400, "new_data_parallel_size must be at least 1")
            if front.spawn is None or front.retire is None:
                return err(400, "this front was started with fixed replicas")
            async with front._lock:
                old = len(front.replicas)
                try:
                    while len(front.replicas) < n:
                        front.replicas.append(await front.spawn(len(front.replicas)))
                    while len(front.replicas) > n:
                        r = front.replicas[-1]
                        deadline = time.monotonic() + float(body.get("drain_timeout", 300))
                        r.healthy = False                      # no new requests; wait for the ones in flight
                        while r.outstanding > 0 and time.monotonic() < deadline:
                            await asyncio.sleep(0.05)
                        front.replicas.pop()
                        await front.retire(r)
                except Exception as e:  # noqa: BLE001
                    return err(500, f"scaling from {old} to {n} stopped at {len(front.replicas)}: {e!r}")
            return {"data_parallel_size": len(front.replicas), "previous": old}

        async def relay(req: Request, path: str):
            body = await req.body()
            pinned = req.headers.get("x-data-parallel-rank")
            await front.revive()
            try:
                r = front.pick(int(pinned) if pinned is not None else None)
            except ValueError as e:
                return err(400, str(e))
            if r is None:
                return err(503, "no data-parallel replica is serving")
            stream = False
            if body and req.headers.get("content-type", "").startswith("application/json"):
                try:
                    stream = bool(json.loads(body).get("stream"))
                except (ValueError, AttributeError):
                    stream = False
            headers = {k: v for k, v in req.headers.items() if k.lower() in ("content-type", "traceparent", "authorization")}
            r.outstanding += 1
            r.served += 1
            if not stream:
                try:
                    resp = await r.client.request(req.method, path, content=body, headers=headers, timeout=None)
                except Exception as e:  # noqa: BLE001
                    r.healthy = False
                    return err(502, f"replica {r.rank} did not answer: {e!r}")
                finally:
                    r.outstanding -= 1
                return Response(resp.content, status_code=resp.status_code,
                                media_type=resp.headers.get("content-type", "application/json"),
                                headers={"x-data-parallel-rank": str(r.rank)})

            async def chunks():
                try:
                    async with r.client.stream(req.method, path, content=body, headers=headers, timeout=None) as resp:
                        async for part in resp.aiter_raw():
                            yield part
                except Exception as e:  # noqa: BLE001
                    r.healthy = False
                    yield ("data: " + json.dumps({"error": {"message": f"replica {r.rank}: {e!r}", "code": 502}})
                           + "\n\ndata: [DONE]\n\n").encode()
                finally:
                    r.outstanding -= 1

            return StreamingResponse(chunks(), media_type="text/event-stream",
                                     headers={"x-data-parallel-rank": str(r.rank)})

        @app.api_route("/{path:path}", methods=["GET", "POST"])
        async def any_route(path: str, req: Request):
            return await relay(req, "/" + path)

        return app


# ---------------------------------------------------------------------- process management (real deployments)
def replica_command(argv: list, port: int) -> list:
    """The ``serve`` command line of one replica: the front's own arguments without the data-parallel size and with
    the private port."""
    out, skip = [], False
    for a in argv:
        if skip:
            skip = False
            continue
        if a in ("--data-parallel-size", "-dp", "--port", "--host"):
            skip = True
            continue
        if a.startswith(("--data-parallel-size=", "--port=", "--host=")):
            continue
        out.append(a)
    return [sys.executable, "-m", "vllm_metax_b200.entrypoints.cli"] + out + ["--port", str(port), "--host", "127.0.0.1"]


def run_front(argv: list, host: str, port: int, dp: int, devices_per_replica: int = 1, on_gpu: bool = True) -> int:
    """Start ``dp`` replica servers, wait until they are healthy, serve the front."""
    import httpx
    import uvicorn

    base = os.environ.get("CUDA_VISIBLE_DEVICES")
    procs: dict = {}

    def visible(rank: int) -> Optional[str]:
        if not on_gpu:
            return None
        ids = base.split(",") if base else [str(i) for i in range((rank + 1) * devices_per_replica)]
        mine = ids[rank * devices_per_replica:(rank + 1) * devices_per_replica]
        if len(mine) < devices_per_replica:
            raise RuntimeError(f"no devices left for replica {rank}")
        return ",".join(mine)

    async def spawn(rank: int) -> Replica:
        p = port + 1 + rank
        env = dict(os.environ, B200_DP_RANK=str(rank))
        v = visible(rank)
        if v is not None:
            env["CUDA_VISIBLE_DEVICES"] = v
        proc = subprocess.Popen(replica_command(argv, p), env=env)
        procs[rank] = proc
        client = httpx.AsyncClient(base_url=f"http://127.0.0.1:{p}")
        r = Replica(rank, f"http://127.0.0.1:{p}", client, proc)
        deadline = time.monotonic() + 1800
        while time.monotonic() < deadline:
            if proc.poll() is not None:
                raise RuntimeError(f"replica {rank} exited with code {proc.returncode} while starting")
            try:
                if (await client.get("/health", timeout=2.0)).status_code == 200:
                    return r
            except Exception:  # noqa: BLE001
                pass
            await asyncio.sleep(0.5)
        proc.terminate()
        raise RuntimeError(f"replica {rank} did not become healthy")

    async def retire(r: Replica) -> None:
        await r.client.aclose()
        if r.proc is not None:
            r.proc.terminate()
            try:
                r.proc.wait(timeout=30)
            except subprocess.TimeoutExpired:
                r.proc.kill()
        procs.pop(r.rank, None)

    async def main() -> None:
        replicas = await asyncio.gather(*[spawn(i) for i in range(dp)])
        front = DataParallelFront(list(replicas), spawn, retire)
        server = uvicorn.Server(uvicorn.Config(front.build_app(), host=host, port=port, log_level="info"))
        try:
            await server.serve()
        finally:
            for r in list(front.replicas):
                await retire(r)

    # The HTTP server restores the previous handlers when it stops and raises the signal it caught again; the default
    # action would end this process before the replicas are retired.  A handler that raises SystemExit lets the
    # ``finally`` blocks run.
    import signal

    def leave(signum, _frame):
        raise SystemExit(128 + signum)

    for sig in (signal.SIGTERM, signal.SIGINT):
        signal.signal(sig, leave)
    try:
        asyncio.run(main())
    except SystemExit:
        pass
    finally:
        left = [proc for proc in procs.values() if proc.poll() is None]      # exactly the processes started above
        for proc in left:
            proc.terminate()
        for proc in left:
            try:
                proc.wait(timeout=30)
            except subprocess.TimeoutExpired:
                proc.kill()
    return 0
