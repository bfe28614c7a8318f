"""Per-kernel time tables from a torch-profiler run of the engine.

    python -m vllm_metax_b200.tools.profile_tables --model '{...}' --num-prompts 8 --input-len 256 --output-len 16

Runs the workload under ``torch.profiler`` (CUDA activities), groups device kernels by name and prints count,
total / mean time and share - the quick "where does a step go" view.  ``LLM.start_profile`` / ``stop_profile``
write a full trace for TensorBoard; this prints the summary without leaving the terminal.
Parity: the reference's profiling docs (docs/developing/msprobe, the torch-profiler hooks of upstream vLLM).
"""
from __future__ import annotations

import argparse
import json
from collections import defaultdict


def kernel_table(events, top: int = 30) -> list[dict]:
    agg: dict[str, list[float]] = defaultdict(list)
    for e in events:
        dev_us = getattr(e, "device_time_total", None)
        if dev_us is None:
            dev_us = getattr(e, "cuda_time_total", 0.0)
        if dev_us and getattr(e, "device_type", None) is not None and "CUDA" in str(e.device_type):
            agg[e.name].append(float(dev_us))
    total = sum(sum(v) for v in agg.values()) or 1.0
    rows = [{"kernel": k, "count": len(v), "total_us": round(sum(v), 1), "mean_us": round(sum(v) / len(v), 2),
             "share": round(sum(v) / total, 4)} for k, v in agg.items()]
    rows.sort(key=lambda r: -r["total_us"])
    return rows[:top]


def format_table(rows: list[dict]) -> str:
    lines = [f"{'share':>7} {'total_us':>12} {'count':>7} {'mean_us':>10}  kernel"]
    for r in rows:
        lines.append(f"{r['share'] * 100:6.2f}% {r['total_us']:12.1f} {r['count']:7d} {r['mean_us']:10.2f}  {r['kernel'][:110]}")
    return "\n".join(lines)


def main(argv=None) -> int:
    import torch

    from .. import LLM, SamplingParams

    ap = argparse.ArgumentParser()
    ap.add_argument("--model", required=True)
    ap.add_argument("--num-prompts", type=int, default=8)
    ap.add_argument("--input-len", type=int, default=256)
    ap.add_argument("--output-len", type=int, default=16)
    ap.add_argument("--tensor-parallel-size", type=int, default=1)
    ap.add_argument("--load-format", default="dummy")
    ap.add_argument("--top", type=int, default=30)
    ap.add_argument("--json", action="store_true")
    a = ap.parse_args(argv)
    model = json.loads(a.model) if a.model.strip().startswith("{") else a.model
    llm = LLM(model, tensor_parallel_size=a.tensor_parallel_size, load_format=a.load_format, enforce_eager=True)
    vocab = llm.engine.cfg.model.vocab_size
    g = torch.Generator().manual_seed(0)
    prompts = [torch.randint(3, vocab, (a.input_len,), generator=g).tolist() for _ in range(a.num_prompts)]
    sp = SamplingParams(max_tokens=a.output_len, temperature=0.0, ignore_eos=True)
    llm.generate(prompts[:1], sp)                       # warm-up outside the profile
    acts = [torch.profiler.ProfilerActivity.CPU]
    if torch.cuda.is_available():
        acts.append(torch.profiler.ProfilerActivity.CUDA)
    with torch.profiler.profile(activities=acts) as prof:
        llm.generate(prompts, sp)
        if torch.cuda.is_available():
            torch.cuda.synchronize()
    rows = kernel_table(prof.events(), a.top)
    print(json.dumps(rows) if a.json else format_table(rows))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
