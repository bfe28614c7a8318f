"""Offline generation with random weights (no checkpoint needed): python examples/offline_inference.py [--device cpu]"""
import argparse

import torch

from vllm_metax_b200 import LLM, SamplingParams

ap = argparse.ArgumentParser()
ap.add_argument("--device", default="cuda" if torch.cuda.is_available() else "cpu")
a = ap.parse_args()
cfg = {"architectures": ["LlamaForCausalLM"], "vocab_size": 1024, "hidden_size": 256, "intermediate_size": 512,
       "num_hidden_layers": 2, "num_attention_heads": 4, "num_key_value_heads": 2, "head_dim": 64,
       "torch_dtype": "float32" if a.device == "cpu" else "bfloat16"}
llm = LLM(cfg, device=a.device, load_format="dummy", max_model_len=256, block_size=16 if a.device == "cpu" else 64,
          num_gpu_blocks=64)
outs = llm.generate([[1, 2, 3, 4, 5], [7, 8, 9]], SamplingParams(max_tokens=8, temperature=0.0, ignore_eos=True))
for o in outs:
    print(o.request_id, o.outputs[0].token_ids)
