"""Command line: ``b200-serve serve <model> [...]``, ``b200-serve bench ...``, ``b200-serve collect-env``.

``serve`` starts the OpenAI-compatible server (single process per node rank 0; tensor-parallel ranks are
started by ``torchrun`` and run the same engine SPMD - only rank 0 binds the port).
Parity: ``vllm serve`` / ``vllm bench serve`` usage in the reference's docs (docs/getting_started/quickstart.md)."""
from __future__ import annotations

import argparse
import json
import sys


def build_parser() -> argparse.ArgumentParser:
    p = argparse.ArgumentParser(prog="b200-serve")
    sub = p.add_subparsers(dest="cmd", required=True)
    s = sub.add_parser("serve", help="start the OpenAI-compatible server")
    s.add_argument("model", help="HF checkpoint directory, or a JSON file / string with a model config")
    s.add_argument("--host", default="0.0.0.0")
    s.add_argument("--port", type=int, default=8000)
    s.add_argument("--served-model-name", default=None)
    s.add_argument("--tensor-parallel-size", "-tp", type=int, default=1)
    s.add_argument("--data-parallel-size", "-dp", type=int, default=1,
                   help="N single-GPU engine servers on ports port+1.. behind one balancing front on --port")
    s.add_argument("--dtype", default="bfloat16")
    s.add_argument("--kv-cache-dtype", default="auto")
    s.add_argument("--max-model-len", type=int, default=4096)
    s.add_argument("--max-num-seqs", type=int, default=256)
    s.add_argument("--max-num-batched-tokens", type=int, default=8192)
    s.add_argument("--gpu-memory-utilization", type=float, default=0.8)
    s.add_argument("--block-size", type=int, default=64)
    s.add_argument("--load-format", default="auto", choices=["auto", "dummy", "safetensors", "sharded_state"])
    s.add_argument("--enable-prefix-caching", action="store_true")
    s.add_argument("--scheduling-policy", default="fcfs", choices=["fcfs", "priority"],
                   help="priority: requests carry a 'priority' (smaller first) and the least important is pre-empted first")
    s.add_argument("--enable-sleep-mode", action="store_true")
    s.add_argument("--enforce-eager", action="store_true")
    s.add_argument("--device", default="cuda")
    s.add_argument("--seed", type=int, default=0)
    s.add_argument("--otlp-traces-endpoint", default=None, help="OTLP/HTTP collector, e.g. http://localhost:4318")
    s.add_argument("--enable-lora", action="store_true")
    s.add_argument("--max-loras", type=int, default=4)
    s.add_argument("--max-lora-rank", type=int, default=64)
    s.add_argument("--lora-modules", nargs="*", default=[], metavar="NAME=PATH", help="PEFT adapters served under NAME")
    s.add_argument("--tool-call-parser", default=None,
                   help="hermes | qwen | llama3_json | llama4_json | llama4_pythonic | mistral | deepseek_v3 | deepseek_v31 | "
                        "pythonic | granite | granite-20b-fc | internlm | phi4_mini_json | minimax | hunyuan_a13b | jamba | "
                        "xlam | kimi_k2 | qwen3_coder | glm45")
    s.add_argument("--enable-auto-tool-choice", action="store_true", help="accepted for command-line compatibility: "
                   "tool_choice=auto is served whenever a tool-call parser is set")
    s.add_argument("--reasoning-parser", default=None, help="deepseek_r1 | qwen3 | glm45 | step3 | mistral | granite | hunyuan_a13b")
    s.add_argument("--chat-template", default=None, help="Jinja chat template: a file (examples/chat_templates/) or "
                   "the template text; replaces the tokenizer's own")
    s.add_argument("--kv-transfer-config", default=None, help="JSON, e.g. '{\"kv_connector\": \"SharedStorageConnector\", "
                   "\"kv_role\": \"kv_producer\", \"kv_connector_extra_config\": {\"shared_storage_path\": \"/dev/shm/kv\"}}'")
    b = sub.add_parser("bench", help="offline throughput / latency run (same engine, no HTTP)")
    b.add_argument("model")
    b.add_argument("--num-prompts", type=int, default=64)
    b.add_argument("--input-len", type=int, default=1024)
    b.add_argument("--output-len", type=int, default=128)
    b.add_argument("--tensor-parallel-size", "-tp", type=int, default=1)
    b.add_argument("--load-format", default="dummy")
    b.add_argument("--device", default="cuda")
    sub.add_parser("collect-env", help="print the environment report")
    return p


def _model_arg(model: str):
    if model.strip().startswith("{"):
        return json.loads(model)
    if model.endswith(".json"):
        with open(model) as f:
            return json.load(f)
    return model


def make_llm(args):
    import torch

    from ..engine.llm import LLM

    kw = dict(tensor_parallel_size=args.tensor_parallel_size, load_format=args.load_format, device=args.device)
    for name in ("max_model_len", "max_num_seqs", "max_num_batched_tokens", "gpu_memory_utilization", "block_size",
                 "enable_prefix_caching", "enable_sleep_mode", "enforce_eager", "kv_cache_dtype", "seed",
                 "scheduling_policy"):
        if hasattr(args, name):
            kw[name] = getattr(args, name)
    if getattr(args, "enable_lora", False):
        kw.update(enable_lora=True, max_loras=args.max_loras, max_lora_rank=args.max_lora_rank)
    if getattr(args, "kv_transfer_config", None):
        kw["kv_transfer_config"] = json.loads(args.kv_transfer_config)
    if hasattr(args, "dtype"):
        kw["dtype"] = {"bfloat16": torch.bfloat16, "float16": torch.float16, "float32": torch.float32}[args.dtype]
    return LLM(_model_arg(args.model), **kw)


def main(argv=None) -> int:
    args = build_parser().parse_args(argv)
    if args.cmd == "collect-env":
        from ..collect_env import main as ce

        ce()
        return 0
    if args.cmd == "bench":
        import time

        import torch

        from ..engine.sampling_params import SamplingParams

        llm = make_llm(args)
        vocab = llm.engine.cfg.model.vocab_size
        g = torch.Generator().manual_seed(0)
        prompts = [torch.randint(0, vocab, (args.input_len,), generator=g).tolist() for _ in range(args.num_prompts)]
        sp = SamplingParams(max_tokens=args.output_len, ignore_eos=True)
        t0 = time.perf_counter()
        outs = llm.generate(prompts, sp)
        dt = time.perf_counter() - t0
        n_out = sum(len(o.outputs[0].token_ids) for o in outs)
        print(json.dumps({"requests": len(outs), "seconds": dt, "output_tok_s": n_out / dt,
                          "total_tok_s": (n_out + args.input_len * len(outs)) / dt}))
        return 0
    # serve
    if getattr(args, "data_parallel_size", 1) > 1:
        if args.tensor_parallel_size > 1:
            raise SystemExit("--data-parallel-size replicas are single-GPU processes; for tensor-parallel replicas "
                             "start one torchrun server per group and balance in front of them")
        from .dp_front import run_front

        return run_front(list(argv if argv is not None else sys.argv[1:]), args.host, args.port, args.data_parallel_size,
                         on_gpu=args.device != "cpu")
    import uvicorn

    from ..parallel import state as ps
    from .async_engine import AsyncLLM
    from .openai_server import build_app

    llm = make_llm(args)
    if ps.global_rank() != 0:
        raise SystemExit("tensor-parallel serving runs the HTTP front on rank 0 only; start ranks with torchrun")
    from ..lora import LoRARequest

    loras = {n: LoRARequest(n, i + 1, p) for i, (n, p) in enumerate(m.split("=", 1) for m in args.lora_modules)}
    from ..utils.observability import RequestTracer

    name = args.served_model_name or str(args.model)
    app = build_app(AsyncLLM(llm, RequestTracer.from_endpoint(args.otlp_traces_endpoint, name)), name, loras,
                    tool_call_parser=args.tool_call_parser, reasoning_parser=args.reasoning_parser,
                    chat_template=args.chat_template)
    uvicorn.run(app, host=args.host, port=args.port, log_level="info")
    return 0


if __name__ == "__main__":
    sys.exit(main())
