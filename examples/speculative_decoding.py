"""N-gram speculative decoding gives the same tokens in fewer engine steps: python examples/speculative_decoding.py"""
import torch

from vllm_metax_b200 import LLM, SamplingParams

dev = "cuda" if torch.cuda.is_available() else "cpu"
cfg = {"architectures": ["LlamaForCausalLM"], "vocab_size": 32, "hidden_size": 64, "intermediate_size": 128,
       "num_hidden_layers": 2, "num_attention_heads": 4, "num_key_value_heads": 2, "head_dim": 16,
       "torch_dtype": "float32" if dev == "cpu" else "bfloat16"}
kw = dict(device=dev, load_format="dummy", max_model_len=256, block_size=16, num_gpu_blocks=64)
sp = SamplingParams(max_tokens=48, temperature=0.0, ignore_eos=True)
prompt = [[1, 2, 3, 1, 2, 3, 1, 2]]
plain = LLM(cfg, **kw)
spec = LLM(cfg, speculative_config={"method": "ngram", "num_speculative_tokens": 4}, **kw)
a, b = plain.generate(prompt, sp), spec.generate(prompt, sp)
assert a[0].outputs[0].token_ids == b[0].outputs[0].token_ids
print("steps:", plain.engine.stats["steps"], "->", spec.engine.stats["steps"],
      "accepted", spec.engine.stats["accepted_tokens"], "of", spec.engine.stats["draft_tokens"], "drafts")
