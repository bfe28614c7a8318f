from __future__ import annotations

from dataclasses import dataclass
from typing import Optional


@dataclass(frozen=True)
class LoRARequest:
    """Names one adapter.  ``lora_int_id`` > 0 identifies it inside the engine (prefix-cache keys, slots);
    ``lora_path`` is a PEFT directory (``adapter_config.json`` + ``adapter_model.safetensors``), or ``tensors`` /
    ``config`` give the same content in memory."""
    lora_name: str
    lora_int_id: int
    lora_path: Optional[str] = None
    tensors: Optional[object] = None          # dict name -> tensor (PEFT naming); not hashed
    config: Optional[object] = None           # dict with r / lora_alpha

    def __post_init__(self):
        if self.lora_int_id < 1:
            raise ValueError("lora_int_id must be >= 1")

    def __hash__(self):
        return hash((self.lora_name, self.lora_int_id))

    def __eq__(self, other):
        return isinstance(other, LoRARequest) and (self.lora_name, self.lora_int_id) == (other.lora_name, other.lora_int_id)
