"""The data-parallel HTTP front over in-process replica applications: balancing by outstanding requests, pinning by
header, relayed streams, a replica that fails is taken out of rotation, elastic scaling, merged metrics."""
import asyncio
import json
import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

httpx = pytest.importorskip("httpx")

from vllm_metax_b200.entrypoints.dp_front import DataParallelFront, Replica, replica_command  # noqa: E402


def _backend():
    """A stand-in for one engine server (the front is what is under test; two real engines do not share a process):
    the same routes, a deterministic answer, 20 ms per request so that concurrent requests overlap."""
    from fastapi import FastAPI, Request
    from fastapi.responses import PlainTextResponse, StreamingResponse

    app = FastAPI()
    state = {"requests": 0}

    @app.get("/health")
    async def health():
        return {}

    @app.get("/metrics")
    async def metrics():
        return PlainTextResponse(f"# HELP x\nb200:requests_total {state['requests']}\n"
                                 f"b200:latency_bucket{{le=\"1\"}} 3\n")

    @app.get("/v1/models")
    async def models():
        return {"data": [{"id": "toy"}]}

    @app.post("/v1/completions")
    async def completions(req: Request):
        body = await req.json()
        state["requests"] += 1
        await asyncio.sleep(0.02)
        toks = [(len(body["prompt"]) * 7 + i) % 251 for i in range(body["max_tokens"])]
        if body.get("stream"):
            async def sse():
                for t in toks:
                    yield "data: " + json.dumps({"choices": [{"text": chr(97 + t % 26), "token_ids": [t]}]}) + "\n\n"
                    await asyncio.sleep(0.001)
                yield "data: [DONE]\n\n"
            return StreamingResponse(sse(), media_type="text/event-stream")
        return {"choices": [{"index": 0, "text": "".join(chr(97 + t % 26) for t in toks), "token_ids": toks}]}

    return None, app


def test_replica_command_line():
    cmd = replica_command(["serve", "m", "--data-parallel-size", "4", "--port=8000", "--max-model-len", "64", "-dp", "2"], 8003)
    assert cmd[-4:] == ["--port", "8003", "--host", "127.0.0.1"]
    assert "--data-parallel-size" not in cmd and "-dp" not in cmd and "--port=8000" not in cmd
    assert cmd[3:8] == ["serve", "m", "--max-model-len", "64", "--port"]


def test_front_balances_relays_and_scales():
    backends = [_backend() for _ in range(3)]
    dead = {"on": False}

    class Broken(httpx.AsyncBaseTransport):
        def __init__(self, inner):
            self.inner = inner

        async def handle_async_request(self, request):
            if dead["on"]:
                raise httpx.ConnectError("replica is gone")
            return await self.inner.handle_async_request(request)

    def client(i):
        t = httpx.ASGITransport(app=backends[i][1])
        return httpx.AsyncClient(transport=Broken(t) if i == 1 else t, base_url="http://replica")

    async def go():
        spare = []

        async def spawn(rank):
            r = Replica(rank, "http://replica", client(rank))
            spare.append(rank)
            return r

        async def retire(r):
            await r.client.aclose()

        front = DataParallelFront([Replica(i, "http://replica", client(i)) for i in range(2)], spawn, retire)
        DataParallelFront.PROBE_EVERY_S = 0.0
        app = front.build_app()
        async with httpx.AsyncClient(transport=httpx.ASGITransport(app=app), base_url="http://front") as c:
            body = {"prompt": "hello there", "max_tokens": 6}
            want = (await c.post("/v1/completions", json=body)).json()["choices"][0]["token_ids"]
            # concurrent requests spread over both replicas, answers identical
            rs = await asyncio.gather(*[c.post("/v1/completions", json=body) for _ in range(8)])
            assert all(r.status_code == 200 and r.json()["choices"][0]["token_ids"] == want for r in rs)
            ranks = [r.headers["x-data-parallel-rank"] for r in rs]
            assert set(ranks) == {"0", "1"}
            # pinning
            r = await c.post("/v1/completions", json=body, headers={"X-data-parallel-rank": "1"})
            assert r.headers["x-data-parallel-rank"] == "1"
            assert (await c.post("/v1/completions", json=body, headers={"X-data-parallel-rank": "7"})).status_code == 400
            # streaming is relayed
            text = ""
            async with c.stream("POST", "/v1/completions", json=dict(body, stream=True)) as resp:
                async for line in resp.aiter_lines():
                    if line.startswith("data: ") and line != "data: [DONE]":
                        text += json.loads(line[6:])["choices"][0]["text"]
            assert len(text) == 6
            # other routes pass through
            assert (await c.get("/v1/models")).json()["data"][0]["id"] == "toy"
            m = (await c.get("/metrics")).text
            assert 'replica="0"' in m and 'replica="1"' in m and "b200:dp_front_replicas 2" in m
            # replica 1 stops answering: one request fails over to 502, then everything goes to replica 0
            dead["on"] = True
            codes = [(await c.post("/v1/completions", json=body, headers={"X-data-parallel-rank": "1"})).status_code]
            assert codes == [502]
            rs = [await c.post("/v1/completions", json=body) for _ in range(4)]
            assert all(r.status_code == 200 and r.headers["x-data-parallel-rank"] == "0" for r in rs)
            assert (await c.get("/health")).json() == {"replicas": 2, "healthy": 1}
            dead["on"] = False                       # it comes back and is probed into rotation again
            assert (await c.get("/health")).json()["healthy"] == 2
            # elastic scaling
            r = await c.post("/scale_elastic_ep", json={"new_data_parallel_size": 3})
            assert r.json() == {"data_parallel_size": 3, "previous": 2} and spare == [2]
            rs = await asyncio.gather(*[c.post("/v1/completions", json=body) for _ in range(9)])
            assert {r.headers["x-data-parallel-rank"] for r in rs} == {"0", "1", "2"}
            r = await c.post("/scale_elastic_ep", json={"new_data_parallel_size": 1})
            assert r.json()["data_parallel_size"] == 1
            rs = [await c.post("/v1/completions", json=body) for _ in range(3)]
            assert all(r.headers["x-data-parallel-rank"] == "0" for r in rs)
            assert (await c.post("/scale_elastic_ep", json={"new_data_parallel_size": 0})).status_code == 400
        for r in front.replicas:
            await r.client.aclose()

    asyncio.run(go())


def test_front_with_real_replica_processes():
    """``b200-serve serve ... --data-parallel-size 2`` on CPU: two engine server processes behind the front, requests
    answered through it, one replica retired on request, everything gone after the front is terminated."""
    import subprocess
    import time

    port = 18100 + (os.getpid() % 500) * 3
    cfg = json.dumps({"architecture": "LlamaForCausalLM", "vocab_size": 256, "hidden_size": 64, "intermediate_size": 128,
                      "num_hidden_layers": 2, "num_attention_heads": 4, "num_key_value_heads": 2, "head_dim": 16,
                      "max_position_embeddings": 256})
    front = subprocess.Popen([sys.executable, "-m", "vllm_metax_b200.entrypoints.cli", "serve", cfg, "--device", "cpu",
                              "--load-format", "dummy", "--dtype", "float32", "--port", str(port), "--host", "127.0.0.1",
                              "--data-parallel-size", "2", "--max-model-len", "128", "--block-size", "16"],
                             cwd=ROOT, stdout=subprocess.DEVNULL, stderr=subprocess.DEVNULL)
    base = f"http://127.0.0.1:{port}"
    try:
        deadline = time.monotonic() + 240
        healthy = None
        while time.monotonic() < deadline and front.poll() is None:
            try:
                r = httpx.get(base + "/health", timeout=2)
                if r.status_code == 200:
                    healthy = r.json()
                    break
            except httpx.HTTPError:
                pass
            time.sleep(1)
        assert healthy == {"replicas": 2, "healthy": 2}, (healthy, front.poll())
        outs = [httpx.post(base + "/v1/completions", json={"prompt": [1, 2, 3, 4], "max_tokens": 5}, timeout=120) for _ in range(4)]
        assert all(o.status_code == 200 for o in outs)
        assert len({tuple(o.json()["choices"][0]["token_ids"]) for o in outs}) == 1           # same model on every replica
        assert {o.headers["x-data-parallel-rank"] for o in outs} == {"0", "1"}                # ties go to the idler one
        r = httpx.post(base + "/scale_elastic_ep", json={"new_data_parallel_size": 1}, timeout=120)
        assert r.json() == {"data_parallel_size": 1, "previous": 2}
        assert httpx.get(base + "/health", timeout=5).json() == {"replicas": 1, "healthy": 1}
        assert httpx.post(base + "/v1/completions", json={"prompt": [1, 2, 3, 4], "max_tokens": 5}, timeout=120).status_code == 200
    finally:
        front.terminate()                     # the front ends the replica processes it started
        try:
            front.wait(timeout=60)
        except subprocess.TimeoutExpired:
            front.kill()
    for p in (port + 1, port + 2):            # nothing is left listening on the replicas' ports
        with pytest.raises(httpx.HTTPError):
            httpx.get(f"http://127.0.0.1:{p}/health", timeout=2)
