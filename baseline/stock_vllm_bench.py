"""Comparison row: stock upstream vLLM (the library installed in the image) on the headline configuration.

    python baseline/stock_vllm_bench.py --steps 2 --warmup 1        # 1 GPU; --tp N for tensor parallel

Llama-3.1-8B architecture with random-initialised weights (``load_format="dummy"``), 256 requests of 1024 uniform-random
prompt tokens and 128 greedy output tokens per pass - the workload ``bench.py`` runs.  Timed end to end around
``LLM.generate`` with a host clock (vLLM's engine core runs in its own process), so the number to compare with is
``bench.py``'s ``e2e.value``.  This is the software stack the reference's Python layer is written against, with NVIDIA's
libraries where the reference has MetaX's; it is not the reference itself (which needs the MACA SDK to build).
"""
import argparse
import json
import os
import tempfile
import time

CONFIG = {"architectures": ["LlamaForCausalLM"], "model_type": "llama", "vocab_size": 128256, "hidden_size": 4096,
          "intermediate_size": 14336, "num_hidden_layers": 32, "num_attention_heads": 32, "num_key_value_heads": 8,
          "head_dim": 128, "hidden_act": "silu", "rms_norm_eps": 1e-5, "rope_theta": 500000.0,
          "max_position_embeddings": 131072, "tie_word_embeddings": False, "torch_dtype": "bfloat16",
          "bos_token_id": 128000, "eos_token_id": 128001, "attention_bias": False, "mlp_bias": False}


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--steps", type=int, default=2)
    ap.add_argument("--warmup", type=int, default=1)
    ap.add_argument("--tp", type=int, default=1)
    ap.add_argument("--batch", type=int, default=256)
    ap.add_argument("--input-len", type=int, default=1024)
    ap.add_argument("--output-len", type=int, default=128)
    a = ap.parse_args()
    import numpy as np
    from vllm import LLM, SamplingParams

    d = tempfile.mkdtemp(prefix="llama31_8b_cfg_")
    with open(os.path.join(d, "config.json"), "w") as f:
        json.dump(CONFIG, f)
    llm = LLM(model=d, load_format="dummy", skip_tokenizer_init=True, dtype="bfloat16", tensor_parallel_size=a.tp,
              max_model_len=2048, max_num_seqs=a.batch, max_num_batched_tokens=8192, gpu_memory_utilization=0.88,
              enable_prefix_caching=False, seed=0)
    sp = SamplingParams(max_tokens=a.output_len, ignore_eos=True, temperature=0.0, detokenize=False)
    rng = np.random.default_rng(0)

    def one_pass():
        prompts = [{"prompt_token_ids": rng.integers(1000, 120000, a.input_len).tolist()} for _ in range(a.batch)]
        t0 = time.perf_counter()
        outs = llm.generate(prompts, sp, use_tqdm=False)
        dt = time.perf_counter() - t0
        assert all(len(o.outputs[0].token_ids) == a.output_len for o in outs)
        return dt

    for _ in range(a.warmup):
        one_pass()
    times = [one_pass() for _ in range(a.steps)]
    ms = 1e3 * sum(times) / len(times)
    import vllm

    print(json.dumps({"impl": f"stock vllm {vllm.__version__}", "metric": "output tok/s, end to end around LLM.generate",
                      "value": round(a.batch * a.output_len / (ms / 1e3), 1), "unit": "tok/s", "ms_per_step": round(ms, 2),
                      "n_gpus": a.tp, "steps": a.steps, "warmup": a.warmup, "dtype": "bf16", "data": "synthetic",
                      "config": {"model": "Llama-3.1-8B", "global_batch": a.batch, "seq_len": a.input_len,
                                 "output_len": a.output_len, "parallelism": f"tp{a.tp}"}}))


if __name__ == "__main__":
    main()
