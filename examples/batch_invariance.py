"""Batch-invariant generation: with B200_BATCH_INVARIANT=1 a request produces the same tokens whether it runs alone
or inside any batch (reproducible evaluation, on-policy RL).  The switch pins every reduction whose order would follow
the batch: unsplit decode attention, one GEMM tile shape without split-K / stream-K, no cascade attention, no fused
tensor-parallel collectives.  (The reference's examples/features/batch_invariance/reproducibility_offline.py.)

    B200_BATCH_INVARIANT=1 python examples/batch_invariance.py <model dir>
"""
import os
import sys

os.environ.setdefault("B200_BATCH_INVARIANT", "1")          # before the package is imported

from vllm_metax_b200 import LLM, SamplingParams  # noqa: E402

model = sys.argv[1] if len(sys.argv) > 1 else "Qwen/Qwen3-8B"
llm = LLM(model, max_model_len=2048)
sp = SamplingParams(max_tokens=64, temperature=0.0)
probe = "Explain why floating-point addition is not associative."
alone = llm.generate([probe], sp)[0].outputs[0].token_ids
filler = [f"Write a haiku about the number {i}." for i in range(31)]
in_batch = llm.generate(filler[:10] + [probe] + filler[10:], sp)[10].outputs[0].token_ids
print("identical:", alone == in_batch)
