"""Release the GPU between generation phases (RLHF co-location): python examples/sleep_mode.py"""
import torch

from vllm_metax_b200 import LLM, SamplingParams

cfg = {"architectures": ["LlamaForCausalLM"], "vocab_size": 1024, "hidden_size": 256, "intermediate_size": 512,
       "num_hidden_layers": 2, "num_attention_heads": 4, "num_key_value_heads": 2, "head_dim": 64}
llm = LLM(cfg, load_format="dummy", enable_sleep_mode=True, max_model_len=256, num_gpu_blocks=64)
sp = SamplingParams(max_tokens=8, temperature=0.0, ignore_eos=True)
before = llm.generate([[1, 2, 3]], sp)[0].outputs[0].token_ids
free0 = torch.cuda.mem_get_info()[0]
llm.sleep(level=1)                 # weights go to pinned host memory, the KV cache is dropped
print("freed MiB:", (torch.cuda.mem_get_info()[0] - free0) >> 20)
llm.wake_up()                      # same virtual addresses: tensors and CUDA graphs stay valid
assert llm.generate([[1, 2, 3]], sp)[0].outputs[0].token_ids == before
