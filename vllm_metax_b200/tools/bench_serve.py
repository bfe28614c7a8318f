"""Load generator for the OpenAI-compatible server (random-token prompts, fixed lengths, bounded concurrency):
the client half of the ``serve`` + ``bench serve`` methodology.

    python -m vllm_metax_b200.tools.bench_serve --base-url http://127.0.0.1:8000 --num-prompts 80 \
        --max-concurrency 16 --input-len 128 --output-len 128

Reports request throughput, output tok/s, and p50 / p99 TTFT, TPOT and ITL, as JSON.  ``--temperature``
defaults to 0 and ``ignore_eos`` is always sent, as in the reference's harness.
Parity: tools/batched_test/bench_sweep.sh:3-14 and model_worker.py:141-196 (``vllm bench serve --dataset-name
random --ignore-eos``), patch/enhancement/chores/bench_serve_args.py:284-292.
"""
from __future__ import annotations

import argparse
import asyncio
import json
import random
import statistics
import time


def percentile(xs: list[float], p: float) -> float:
    if not xs:
        return float("nan")
    xs = sorted(xs)
    k = (len(xs) - 1) * p / 100.0
    lo, hi = int(k), min(int(k) + 1, len(xs) - 1)
    return xs[lo] + (xs[hi] - xs[lo]) * (k - lo)


def summarize(records: list[dict], wall: float) -> dict:
    ok = [r for r in records if r.get("ok")]
    ttft = [r["ttft"] for r in ok]
    tpot = [(r["latency"] - r["ttft"]) / max(r["output_tokens"] - 1, 1) for r in ok if r["output_tokens"] > 1]
    itl = [d for r in ok for d in r["itl"]]
    out_tokens = sum(r["output_tokens"] for r in ok)
    return {
        "completed": len(ok), "failed": len(records) - len(ok), "duration_s": round(wall, 3),
        "request_throughput": round(len(ok) / wall, 3), "output_tok_s": round(out_tokens / wall, 2),
        "total_tok_s": round((out_tokens + sum(r["prompt_tokens"] for r in ok)) / wall, 2),
        "p50_ttft_ms": round(percentile(ttft, 50) * 1e3, 2), "p99_ttft_ms": round(percentile(ttft, 99) * 1e3, 2),
        "mean_ttft_ms": round(statistics.fmean(ttft) * 1e3, 2) if ttft else None,
        "p50_tpot_ms": round(percentile(tpot, 50) * 1e3, 3), "p99_tpot_ms": round(percentile(tpot, 99) * 1e3, 3),
        "p50_itl_ms": round(percentile(itl, 50) * 1e3, 3), "p99_itl_ms": round(percentile(itl, 99) * 1e3, 3),
    }


async def one_request(session, url: str, model: str, prompt_ids: list[int], out_len: int, temperature: float) -> dict:
    body = {"model": model, "prompt": prompt_ids, "max_tokens": out_len, "temperature": temperature,
            "ignore_eos": True, "stream": True}
    t0 = time.perf_counter()
    first = last = None
    itl: list[float] = []
    n = 0
    try:
        async with session.post(url + "/v1/completions", json=body) as resp:
            if resp.status != 200:
                return {"ok": False, "error": f"http {resp.status}"}
            async for raw in resp.content:
                line = raw.decode().strip()
                if not line.startswith("data: ") or line == "data: [DONE]":
                    continue
                ev = json.loads(line[6:])
                if "error" in ev:
                    return {"ok": False, "error": ev["error"].get("message")}
                k = sum(len(c.get("token_ids") or []) for c in ev.get("choices", []))
                if k == 0:
                    continue
                now = time.perf_counter()
                if first is None:
                    first = now
                else:
                    itl.append(now - last)
                last = now
                n += k
    except Exception as e:  # connection errors count as failed requests
        return {"ok": False, "error": repr(e)}
    t1 = time.perf_counter()
    return {"ok": first is not None, "ttft": (first or t1) - t0, "latency": t1 - t0, "output_tokens": n,
            "prompt_tokens": len(prompt_ids), "itl": itl}


async def run(base_url: str, model: str, num_prompts: int, max_concurrency: int, input_len: int, output_len: int,
              vocab: int, temperature: float, seed: int) -> dict:
    import aiohttp

    rng = random.Random(seed)
    prompts = [[rng.randrange(10, vocab) for _ in range(input_len)] for _ in range(num_prompts)]
    sem = asyncio.Semaphore(max_concurrency)
    timeout = aiohttp.ClientTimeout(total=6 * 3600)
    async with aiohttp.ClientSession(timeout=timeout) as session:
        async def guarded(p):
            async with sem:
                return await one_request(session, base_url, model, p, output_len, temperature)

        t0 = time.perf_counter()
        records = await asyncio.gather(*[guarded(p) for p in prompts])
        wall = time.perf_counter() - t0
    out = summarize(list(records), wall)
    out.update(num_prompts=num_prompts, max_concurrency=max_concurrency, input_len=input_len, output_len=output_len)
    return out


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--base-url", default="http://127.0.0.1:8000")
    ap.add_argument("--model", default="b200-model")
    ap.add_argument("--num-prompts", type=int, default=20)
    ap.add_argument("--max-concurrency", type=int, default=4)
    ap.add_argument("--input-len", type=int, default=1024)
    ap.add_argument("--output-len", type=int, default=1024)
    ap.add_argument("--vocab-size", type=int, default=32000)
    ap.add_argument("--temperature", type=float, default=0.0)
    ap.add_argument("--seed", type=int, default=0)
    a = ap.parse_args(argv)
    res = asyncio.run(run(a.base_url, a.model, a.num_prompts, a.max_concurrency, a.input_len, a.output_len,
                          a.vocab_size, a.temperature, a.seed))
    print(json.dumps(res))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
