"""Beam search, prompt log-probabilities (perplexity) and several samples per prompt, offline.

    python examples/beam_search_and_scoring.py <model dir>
"""
import math
import sys

from vllm_metax_b200 import LLM, SamplingParams

model = sys.argv[1] if len(sys.argv) > 1 else "Qwen/Qwen3-8B"
llm = LLM(model, max_model_len=2048, enable_prefix_caching=True)      # beams and samples share their prompt's cache

# beam search: the 4 most likely 32-token continuations, best first
for beam in llm.beam_search(["The three laws of robotics are"], beam_width=4, max_tokens=32)[0]:
    print(f"{beam['cum_logprob']:8.2f}  {beam['text']!r}")

# perplexity of a text: the log-probability of every token given the ones before it
text = "The quick brown fox jumps over the lazy dog."
entries = llm.prompt_logprobs([text], top=0)[0][1:]                    # the first token has no prediction
print("perplexity:", math.exp(-sum(e["logprob"] for e in entries) / len(entries)))

# independent samples of one prompt, with the log-probability of each generated token
out = llm.generate(["Write a one-line poem about GPUs."], SamplingParams(max_tokens=24, temperature=0.9, n=3, seed=0, logprobs=0))[0]
for c in out.outputs:
    print(c.index, sum(e["logprob"] for e in c.logprobs), repr(c.text))

# stop strings and banned words
sp = SamplingParams(max_tokens=64, temperature=0.0, stop=["\n\n", "User:"], bad_words=["GPU"])
print(repr(llm.generate(["Q: What runs CUDA kernels?\nA:"], sp)[0].outputs[0].text))
