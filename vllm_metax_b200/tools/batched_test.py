"""Batched model test harness: walk a model matrix (``configs/models.yaml``), and for every entry run a
generation smoke test and a benchmark sweep (``configs/bench_*.json``) through the engine, writing one JSON
line per (model, test, sweep point) to a results file.

    python -m vllm_metax_b200.tools.batched_test --models configs/models.yaml --bench configs/bench_default.json \
        --only tiny-llama-dummy --out results.jsonl [--device cpu]

Each model runs in its own process (a crash or an out-of-memory of one entry does not end the sweep); entries
with ``tp > 1`` are launched with ``torch.distributed.run``.  Missing checkpoints are reported as skipped.
Parity: tools/batched_test/ of the reference (README.md:103-131 defaults, model.yaml matrix of 81 models,
model_worker.py:141-196 serve + bench sweep, bench_params/*.json sweep points).
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import time

HERE = os.path.dirname(os.path.abspath(__file__))


def load_matrix(path: str) -> tuple[dict, list[dict]]:
    import yaml

    with open(path) as f:
        doc = yaml.safe_load(f)
    return doc.get("defaults") or {}, doc.get("models") or []


def worker(entry: dict, defaults: dict, sweep: list[dict], device: str) -> list[dict]:
    """Runs inside the child process: build the engine once, run the entry's tests."""
    import torch

    from .. import LLM, SamplingParams

    kw = dict(tensor_parallel_size=int(entry.get("tp", 1)), device=device,
              load_format=entry.get("load_format", "auto"),
              max_model_len=int(entry.get("max_model_len", defaults.get("max_model_len", 4096))),
              gpu_memory_utilization=float(entry.get("gpu_memory_utilization", defaults.get("gpu_memory_utilization", 0.8))),
              enable_expert_parallel=bool(entry.get("enable_expert_parallel", False)),
              kv_cache_dtype=entry.get("kv_cache_dtype", "auto"))
    if device == "cpu":
        kw.update(dtype=torch.float32, num_gpu_blocks=256, block_size=16)
    model = entry["model"]
    llm = LLM(model, **kw)
    vocab = llm.engine.cfg.model.vocab_size
    out = []
    g = torch.Generator().manual_seed(0)
    if "generate" in entry.get("tests", ["generate"]):
        prompts = [torch.randint(3, vocab, (n,), generator=g).tolist() for n in (5, 17, 33)]
        t0 = time.perf_counter()
        res = llm.generate(prompts, SamplingParams(max_tokens=8, temperature=0.0, ignore_eos=True))
        ok = all(len(r.outputs[0].token_ids) == 8 for r in res)
        out.append({"model": entry["name"], "test": "generate", "ok": ok, "seconds": round(time.perf_counter() - t0, 3)})
    if "bench" in entry.get("tests", []):
        max_len = kw["max_model_len"]
        for pt in sweep:
            il, ol = int(pt["input_len"]), int(pt["output_len"])
            if il + ol > max_len:
                out.append({"model": entry["name"], "test": "bench", "skipped": "exceeds max_model_len", **pt})
                continue
            n = int(pt["num_prompts"])
            prompts = [torch.randint(3, vocab, (il,), generator=g).tolist() for _ in range(n)]
            t0 = time.perf_counter()
            res = llm.generate(prompts, SamplingParams(max_tokens=ol, temperature=0.0, ignore_eos=True))
            dt = time.perf_counter() - t0
            ttft = sorted(r.metrics.ttft for r in res if r.metrics.ttft is not None)
            tpot = sorted(r.metrics.tpot for r in res if r.metrics.tpot is not None)
            out.append({"model": entry["name"], "test": "bench", **pt, "seconds": round(dt, 3),
                        "output_tok_s": round(n * ol / dt, 2),
                        "p50_ttft_ms": round(ttft[len(ttft) // 2] * 1e3, 2) if ttft else None,
                        "p50_tpot_ms": round(tpot[len(tpot) // 2] * 1e3, 3) if tpot else None})
    return out


def run_entry(entry: dict, defaults: dict, sweep: list[dict], device: str, timeout: int) -> list[dict]:
    model = entry["model"]
    if isinstance(model, str) and not os.path.isdir(model):
        return [{"model": entry["name"], "skipped": f"checkpoint {model} not found"}]
    payload = json.dumps({"entry": entry, "defaults": defaults, "sweep": sweep, "device": device})
    tp = int(entry.get("tp", 1))
    if tp > 1:
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={tp}",
               "--master-addr", "127.0.0.1", "--master-port", str(29500 + os.getpid() % 400), "-m",
               "vllm_metax_b200.tools.batched_test", "--child", payload]
    else:
        cmd = [sys.executable, "-m", "vllm_metax_b200.tools.batched_test", "--child", payload]
    try:
        p = subprocess.run(cmd, capture_output=True, text=True, timeout=timeout)
    except subprocess.TimeoutExpired:
        return [{"model": entry["name"], "error": f"timeout after {timeout}s"}]
    lines = [l for l in p.stdout.splitlines() if l.startswith("RESULT ")]
    if p.returncode != 0 or not lines:
        return [{"model": entry["name"], "error": (p.stderr or p.stdout)[-800:], "returncode": p.returncode}]
    return json.loads(lines[-1][7:])


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--models", default=os.path.join(HERE, "configs", "models.yaml"))
    ap.add_argument("--bench", default=os.path.join(HERE, "configs", "bench_default.json"))
    ap.add_argument("--only", nargs="*", default=None, help="model names to run")
    ap.add_argument("--out", default="batched_test_results.jsonl")
    ap.add_argument("--device", default="cuda")
    ap.add_argument("--timeout", type=int, default=3600)
    ap.add_argument("--child", default=None, help=argparse.SUPPRESS)
    a = ap.parse_args(argv)
    if a.child is not None:
        d = json.loads(a.child)
        res = worker(d["entry"], d["defaults"], d["sweep"], d["device"])
        if int(os.environ.get("RANK", "0")) == 0:
            print("RESULT " + json.dumps(res), flush=True)
        return 0
    defaults, models = load_matrix(a.models)
    with open(a.bench) as f:
        sweep = json.load(f)
    failed = 0
    with open(a.out, "a") as out:
        for entry in models:
            if a.only and entry["name"] not in a.only:
                continue
            for rec in run_entry(entry, defaults, sweep, a.device, a.timeout):
                failed += 1 if ("error" in rec or rec.get("ok") is False) else 0
                out.write(json.dumps(rec) + "\n")
                out.flush()
                print(json.dumps(rec))
    return 1 if failed else 0


if __name__ == "__main__":
    raise SystemExit(main())
