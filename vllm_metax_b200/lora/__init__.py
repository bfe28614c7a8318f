"""Multi-LoRA serving: several low-rank adapters resident at once, chosen per request.

    llm = LLM(model, enable_lora=True, max_loras=4, max_lora_rank=64)
    llm.generate(prompts, sp, lora_request=LoRARequest("sql", 1, "/path/to/peft_adapter"))

``LoRAManager`` attaches to the target linears of a loaded model (``qkv_proj``, ``o_proj``, ``gate_up_proj``,
``down_proj``): every module gets stacked ``A [slots, R, in]`` / ``B [slots, out, R]`` buffers and a forward hook
that adds ``scale * (x A^T) B^T`` for the rows of the batch whose request uses an adapter.  Fused projections stack
their parts along the rank dimension (q | k | v, gate | up) with a block-structured ``B``; tensor-parallel shards
are cut by the module's own weight loader, so column- and row-parallel layers follow the base weights.
Parity: the reference runs upstream's punica LoRA path (``Platform.get_punica_wrapper``,
vllm_metax/patch/bugfix/triton_support/lora_shrink_op.py:30 retunes its shrink kernel).
"""
from .manager import LoRAManager
from .models import LoRAModel
from .request import LoRARequest

__all__ = ["LoRAManager", "LoRAModel", "LoRARequest"]
