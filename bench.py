#!/usr/bin/env python
"""Headline benchmark: output tokens/s of Llama-3.1-8B serving on N GPUs of one node.

Workload (the reference's `vllm bench serve --dataset-name random --ignore-eos` recipe at the
shape named for this build): 256 concurrent requests, each 1024 uniform-random input tokens
and 128 forced output tokens, bf16, random-init weights, TP = N.  `--config` selects one of the
other serving configurations (`qwen3moe`, `dsv32`, `llama70b_int8kv`); the output line names it.

One *step* is one full pass over that workload (prefill of all requests + 127 decode
iterations).  Two measurements per run:

* ``value``  - device-resident replay (`StaticWorkload`): inputs staged on the GPU, decode as
  CUDA-graph replays with a device-side advance kernel; CUDA-event time, max over ranks.
* ``e2e``    - the same workload through the public API (`LLM.generate`): host scheduler,
  per-step pinned-memory H2D of the step inputs and D2H of the sampled tokens.

`python bench.py --gpus N --steps K --warmup W`; for N > 1 launch under torchrun.
`--impl reference` reports that the reference cannot be installed on this machine.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time

BLOCK_SIZE = 128

# The serving configurations named for this build (random-init weights, uniform-random prompt tokens).
# `model` holds ModelConfig fields; `workload` = (requests, input tokens, output tokens); `prefill_tokens` = tokens
# per prefill step of the device-resident replay; `llm` = extra LLM(...) arguments.
CONFIGS = {
    "llama8b": dict(
        label="Llama-3.1-8B", parallelism="tp",
        model=dict(architecture="LlamaForCausalLM", vocab_size=128256, hidden_size=4096, intermediate_size=14336,
                   num_hidden_layers=32, num_attention_heads=32, num_key_value_heads=8, head_dim=128,
                   rms_norm_eps=1e-5, rope_theta=500000.0, max_position_embeddings=8192),
        workload=(256, 1024, 128), prefill_tokens=8192, llm={}),
    "qwen3moe": dict(
        label="Qwen3-30B-A3B-style MoE (128 experts, top-8)", parallelism="ep",
        model=dict(architecture="Qwen3MoeForCausalLM", vocab_size=151936, hidden_size=2048, intermediate_size=6144,
                   num_hidden_layers=48, num_attention_heads=32, num_key_value_heads=4, head_dim=128,
                   rms_norm_eps=1e-6, rope_theta=1000000.0, max_position_embeddings=40960, qk_norm=True,
                   num_experts=128, num_experts_per_tok=8, moe_intermediate_size=768, norm_topk_prob=True),
        workload=(512, 2048, 256), prefill_tokens=8192, llm={}),
    "dsv32": dict(
        label="DeepSeek-V3.2-style MLA + DSA, block-scaled fp8", parallelism="tp+ep",
        model=dict(architecture="DeepseekV32ForCausalLM", vocab_size=129280, hidden_size=7168, intermediate_size=18432,
                   num_hidden_layers=61, num_attention_heads=128, num_key_value_heads=128, rms_norm_eps=1e-6,
                   rope_theta=10000.0, max_position_embeddings=163840, q_lora_rank=1536, kv_lora_rank=512,
                   qk_nope_head_dim=128, qk_rope_head_dim=64, v_head_dim=128, first_k_dense_replace=3,
                   num_experts=256, num_experts_per_tok=8, moe_intermediate_size=2048, n_shared_experts=1,
                   scoring_func="sigmoid", n_group=8, topk_group=4, routed_scaling_factor=2.5, topk_method="noaux_tc",
                   norm_topk_prob=True, index_n_heads=64, index_head_dim=128, index_topk=2048, quantization="fp8",
                   quant_config={"quant_method": "fp8", "weight_block_size": [128, 128]}),
        workload=(128, 8192, 512), prefill_tokens=8192, llm=dict(kv_cache_dtype="fp8_ds_mla"),
        dtype="fp8 e4m3 block-scaled weights (128x128), bf16 activations"),
    "llama70b_int8kv": dict(
        label="Llama-3.1-70B, int8 KV cache (per-token-per-head scales)", parallelism="tp",
        model=dict(architecture="LlamaForCausalLM", vocab_size=128256, hidden_size=8192, intermediate_size=28672,
                   num_hidden_layers=80, num_attention_heads=64, num_key_value_heads=8, head_dim=128,
                   rms_norm_eps=1e-5, rope_theta=500000.0, max_position_embeddings=131072),
        workload=(32, 32768, 1024), prefill_tokens=8192, llm=dict(kv_cache_dtype="int8")),
}


class ClockSampler:
    """Samples SM clocks / throttle reasons with nvidia-smi while the timed region runs."""

    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu = gpu_index
        self.f = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
        self.p = None

    def start(self):
        try:
            self.p = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                       "-lms", "200", "-i", str(self.gpu)], stdout=self.f, stderr=subprocess.DEVNULL)
        except Exception:
            self.p = None

    def stop(self) -> dict:
        if self.p is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.p.terminate()
        try:
            self.p.wait(timeout=5)
        except Exception:
            self.p.kill()
        self.f.flush()
        self.f.seek(0)
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.f.read().splitlines():
            parts = [x.strip() for x in line.split(",")]
            if len(parts) < 9:
                continue
            try:
                sm.append(float(parts[1])); mx.append(float(parts[2]))
            except ValueError:
                continue
            for nm, v in zip(names, parts[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(nm)
        os.unlink(self.f.name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=2)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours")
    ap.add_argument("--config", default="llama8b", choices=sorted(CONFIGS),
                    help="serving configuration (default: the headline Llama-3.1-8B workload)")
    ap.add_argument("--num-reqs", type=int, default=0, help="debug only: override the configuration's request count")
    ap.add_argument("--in-len", type=int, default=0)
    ap.add_argument("--out-len", type=int, default=0)
    ap.add_argument("--layers", type=int, default=0, help="debug only; a reduced model is named as such in the output")
    ap.add_argument("--pp", type=int, default=1,
                    help="pipeline stages (the other gpus / pp ranks of a stage are tensor parallel); the value is then "
                         "the end-to-end number through LLM.generate, device-timed, because the device-resident "
                         "workload driver is tensor-parallel only")
    args = ap.parse_args()
    conf = CONFIGS[args.config]
    MODEL = conf["model"]
    args.num_reqs = args.num_reqs or conf["workload"][0]
    args.in_len = args.in_len or conf["workload"][1]
    args.out_len = args.out_len or conf["workload"][2]
    args.layers = args.layers or MODEL["num_hidden_layers"]
    PREFILL_TOKENS = conf["prefill_tokens"]

    rank = int(os.environ.get("RANK", "0"))
    if args.impl == "reference":
        if rank == 0:
            print(json.dumps({"impl": "reference", "unavailable":
                              "reference needs the MACA SDK (cmake_maca, +metax torch, mcoplib) and setuptools_scm; "
                              "its offline pip install fails at metadata generation on this image"}))
        return

    import torch
    import torch.distributed as dist

    from vllm_metax_b200 import LLM, ModelConfig, SamplingParams
    from vllm_metax_b200 import _custom_ops as ops
    from vllm_metax_b200.engine.static_workload import StaticWorkload
    from vllm_metax_b200.parallel import state as ps

    world = int(os.environ.get("WORLD_SIZE", "1"))
    assert world == args.gpus, f"launch with torchrun --nproc-per-node {args.gpus} (WORLD_SIZE={world})"
    model = dict(MODEL, num_hidden_layers=args.layers)
    N, P, O = args.num_reqs, args.in_len, args.out_len
    assert args.gpus % args.pp == 0
    llm = LLM(ModelConfig(**model, dtype=torch.bfloat16), tensor_parallel_size=args.gpus // args.pp,
              pipeline_parallel_size=args.pp, block_size=BLOCK_SIZE,
              max_model_len=P + O + BLOCK_SIZE, max_num_seqs=N, max_num_batched_tokens=PREFILL_TOKENS,
              num_gpu_blocks=N * ((P + O + BLOCK_SIZE - 1) // BLOCK_SIZE) + 8, device="cuda", **conf["llm"])
    runner = llm.engine.runner
    dev = runner.device

    def barrier():
        if world > 1:
            dist.barrier(device_ids=[dev.index])
        torch.cuda.synchronize()

    def max_over_ranks(x: float) -> float:
        if world == 1:
            return x
        t = torch.tensor([x], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    # ---------------------------------------------------------------- device-resident measurement
    out_tokens = args.steps * N * O
    sampler = ClockSampler(dev.index or 0)
    launches, phases, tp_check, dev_ms = 0, {}, None, 0.0
    if args.pp == 1:
        wl = StaticWorkload(runner, N, P, O, PREFILL_TOKENS)
        wl.capture()
        for _ in range(args.warmup):
            wl.run()
        barrier()
        if rank == 0:
            sampler.start()
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        ev0.record()
        for _ in range(args.steps):
            launches += wl.run()
        ev1.record()
        barrier()
        dev_ms = max_over_ranks(ev0.elapsed_time(ev1))
        clocks = sampler.stop() if rank == 0 else {}
        ops.check_kernel_status(dev.index or 0)
        phases = wl.phase_ms()
        # outside the timed region: the fused NVLink path against the library collectives on the same ranks
        tp_check = wl.collective_check() if world > 1 else None
        value = out_tokens / (dev_ms / 1e3)

    # ---------------------------------------------------------------- end to end through LLM.generate
    g = torch.Generator().manual_seed(1)
    prompts_host = torch.randint(0, model["vocab_size"], (N, P), generator=g).pin_memory()
    prompts = prompts_host.tolist()
    sp = SamplingParams(max_tokens=O, temperature=0.0, ignore_eos=True)
    for _ in range((min(args.warmup, 1) or 1) if args.pp == 1 else args.warmup):
        llm.generate(prompts, sp)
    barrier()
    if args.pp > 1 and rank == 0:
        sampler.start()
    l0 = ops.launch_count()
    runner.h2d_bytes = runner.d2h_bytes = 0
    ttfts, tpots = [], []
    t0 = time.perf_counter()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        outs = llm.generate(prompts, sp)
        ttfts += [o.metrics.ttft for o in outs]
        tpots += [o.metrics.tpot for o in outs]
        assert all(len(o.outputs[0].token_ids) == O for o in outs)
    e1.record()
    barrier()
    e2e_ms = max_over_ranks(max(e0.elapsed_time(e1), (time.perf_counter() - t0) * 1e3))
    e2e_value = out_tokens / (e2e_ms / 1e3)
    ops.check_kernel_status(dev.index or 0)
    if args.pp > 1:          # no device-resident driver for pipeline stages: the end-to-end run is the measurement
        clocks = sampler.stop() if rank == 0 else {}
        dev_ms, value, launches = e2e_ms, e2e_value, ops.launch_count() - l0
        phases = {"note": "timed through LLM.generate", "max_inflight": llm.engine.stats.get("max_inflight", 0)}

    if rank == 0:
        print(json.dumps({
            "metric": f"output tok/s ({conf['label']}, {N} req x {P} in / {O} out, device-timed, max over ranks)",
            "value": round(value, 1), "unit": "tok/s", "n_gpus": args.gpus, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": round(dev_ms / args.steps, 2), "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": conf.get("dtype", "bf16"), "data": "synthetic",
            "impl": "ours",
            "config": {"name": args.config,
                       "model": conf["label"] if args.layers == MODEL["num_hidden_layers"]
                       else f"{conf['label']}[{args.layers} layers, debug]",
                       "global_batch": N, "seq_len": P, "output_len": O,
                       "parallelism": "+".join(f"{x}{args.gpus // args.pp}" for x in conf["parallelism"].split("+"))
                       + (f"+pp{args.pp}" if args.pp > 1 else ""),
                       "block_size": BLOCK_SIZE, "prefill_tokens_per_step": PREFILL_TOKENS,
                       "l2": "inputs larger than L2 (weights + KV cache streamed every iteration)",
                       "step": "one pass over the whole workload (prefill + decode of all requests)",
                       "last_pass_phases_rank0": phases},
            "clocks": clocks,
            "e2e": {"value": round(e2e_value, 1), "unit": "tok/s", "ms_per_step": round(e2e_ms / args.steps, 2),
                    "h2d_bytes_per_step": runner.h2d_bytes // args.steps,
                    "d2h_bytes_per_step": runner.d2h_bytes // args.steps,
                    "p50_ttft_ms": round(statistics.median(ttfts) * 1e3, 2),
                    "p50_tpot_ms": round(statistics.median(tpots) * 1e3, 3)},
            "gpu_launches": launches,
            **({"tp_check": tp_check} if tp_check is not None else {}),
        }))
    if world > 1:
        # release captured graphs before the communicators they reference, and never let a slow
        # NCCL teardown keep a finished benchmark alive
        import threading

        sys.stdout.flush()
        threading.Timer(30.0, lambda: os._exit(0)).start()
        if args.pp == 1:
            wl.graph = None
        runner.graphs.clear()
        torch.cuda.synchronize()
        ps.destroy()
        os._exit(0)


if __name__ == "__main__":
    main()
