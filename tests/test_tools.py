"""Harness tools on CPU: batched test matrix on the dummy model, bench_serve statistics, profiler tables, precision dump."""
import json
import os
import sys

import torch

from vllm_metax_b200 import LLM, ModelConfig, SamplingParams
from vllm_metax_b200.tools import batched_test, bench_serve, profile_tables
from vllm_metax_b200.utils.precision_dump import PrecisionDump, compare_dumps


def test_batched_harness_runs_dummy_entry(tmp_path):
    defaults, models = batched_test.load_matrix(os.path.join(os.path.dirname(batched_test.__file__), "configs", "models.yaml"))
    entry = next(m for m in models if m["name"] == "tiny-llama-dummy")
    sweep = [{"max_concurrency": 1, "num_prompts": 2, "input_len": 16, "output_len": 4}]
    recs = batched_test.run_entry(entry, dict(defaults, max_model_len=128), sweep, "cpu", timeout=600)
    kinds = {r.get("test") for r in recs}
    assert kinds == {"generate", "bench"} and all("error" not in r for r in recs), recs
    assert next(r for r in recs if r["test"] == "bench")["output_tok_s"] > 0
    # a missing checkpoint is a skip, not a failure
    assert "skipped" in batched_test.run_entry({"name": "x", "model": "/no/such/dir"}, defaults, sweep, "cpu", 10)[0]


def test_bench_serve_statistics():
    recs = [{"ok": True, "ttft": 0.1, "latency": 1.1, "output_tokens": 11, "prompt_tokens": 8, "itl": [0.1] * 10},
            {"ok": True, "ttft": 0.3, "latency": 0.8, "output_tokens": 6, "prompt_tokens": 8, "itl": [0.1] * 5},
            {"ok": False, "error": "x"}]
    s = bench_serve.summarize(recs, wall=2.0)
    assert s["completed"] == 2 and s["failed"] == 1 and s["output_tok_s"] == 8.5
    assert abs(s["p50_ttft_ms"] - 200.0) < 1e-6 and abs(s["p50_tpot_ms"] - 100.0) < 1e-6
    assert bench_serve.percentile([1, 2, 3, 4], 50) == 2.5


def test_profile_table_formatting():
    class E:
        def __init__(self, name, us):
            self.name, self.device_time_total, self.device_type = name, us, "DeviceType.CUDA"
    rows = profile_tables.kernel_table([E("a", 10.0), E("a", 30.0), E("b", 60.0)])
    assert rows[0]["kernel"] == "b" and rows[1]["count"] == 2 and abs(rows[1]["share"] - 0.4) < 1e-9
    assert "kernel" in profile_tables.format_table(rows)


def test_precision_dump_finds_first_divergence(tmp_path):
    cfg = ModelConfig(architecture="LlamaForCausalLM", vocab_size=64, hidden_size=64, intermediate_size=128,
                      num_hidden_layers=3, num_attention_heads=4, num_key_value_heads=2, head_dim=16,
                      max_position_embeddings=128, dtype=torch.float32)
    kw = dict(device="cpu", load_format="dummy", num_gpu_blocks=16, block_size=16, max_model_len=64, seed=0)
    sp = SamplingParams(max_tokens=2, temperature=0.0, ignore_eos=True)
    a, b = str(tmp_path / "a.jsonl"), str(tmp_path / "b.jsonl")
    llm = LLM(cfg, **kw)
    model = llm.engine.runner.model
    with PrecisionDump(model, a, pattern=r"layers\.\d+$"):
        llm.generate([[1, 2, 3]], sp)
    with PrecisionDump(model, b, pattern=r"layers\.\d+$"):
        llm.generate([[1, 2, 3]], sp)
    assert compare_dumps(a, b)["mismatches"] == 0
    model.model.layers["1"].mlp.down_proj.weight.data.mul_(3.0)          # break layer 1
    with PrecisionDump(model, b, pattern=r"layers\.\d+$"):
        llm.generate([[1, 2, 3]], sp)
    rep = compare_dumps(a, b)
    assert rep["mismatches"] > 0 and rep["first"]["key"][0] == "model.layers.1"
