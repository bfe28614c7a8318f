"""One adapter's weights, parsed from PEFT naming into per-module (A, B) pairs."""
from __future__ import annotations

import json
import os
import re
from typing import Optional

import torch

# HF projection name -> (module attribute in this package's models, shard id inside a fused module)
TARGETS = {
    "q_proj": ("qkv_proj", "q"), "k_proj": ("qkv_proj", "k"), "v_proj": ("qkv_proj", "v"), "o_proj": ("o_proj", None),
    "gate_proj": ("gate_up_proj", 0), "up_proj": ("gate_up_proj", 1), "down_proj": ("down_proj", None),
}
_KEY = re.compile(r"(?:base_model\.model\.)?(?P<mod>.+)\.(?P<proj>[a-z_]+_proj)\.lora_(?P<ab>[AB])(?:\.default)?\.weight$")


class LoRAModel:
    def __init__(self, rank: int, alpha: float, weights: dict):
        self.rank, self.alpha = rank, alpha
        self.scaling = alpha / rank
        # {(parent module path, fused module name): {shard id: (A [r, in], B [out, r])}}
        self.weights = weights

    @classmethod
    def from_tensors(cls, tensors: dict, config: Optional[dict] = None) -> "LoRAModel":
        pairs: dict = {}
        for name, t in tensors.items():
            m = _KEY.match(name)
            if m is None or m["proj"] not in TARGETS:
                continue
            pairs.setdefault((m["mod"], m["proj"]), {})[m["ab"]] = t
        if not pairs:
            raise ValueError("no LoRA tensors for q/k/v/o/gate/up/down projections found")
        rank = None
        weights: dict = {}
        for (mod, proj), ab in pairs.items():
            if "A" not in ab or "B" not in ab:
                raise ValueError(f"adapter is missing lora_A or lora_B of {mod}.{proj}")
            a, b = ab["A"].float(), ab["B"].float()
            if a.shape[0] != b.shape[1]:
                raise ValueError(f"rank mismatch in {mod}.{proj}: A {tuple(a.shape)} vs B {tuple(b.shape)}")
            rank = a.shape[0] if rank is None else rank
            if a.shape[0] != rank:
                raise ValueError("adapters with per-module ranks are not supported")
            fused, shard = TARGETS[proj]
            weights.setdefault((mod, fused), {})[shard] = (a, b)
        alpha = float((config or {}).get("lora_alpha", rank))
        return cls(int(rank), alpha, weights)

    @classmethod
    def from_peft_dir(cls, path: str) -> "LoRAModel":
        with open(os.path.join(path, "adapter_config.json")) as f:
            config = json.load(f)
        st = os.path.join(path, "adapter_model.safetensors")
        if os.path.exists(st):
            from safetensors.torch import load_file

            tensors = load_file(st)
        else:
            tensors = torch.load(os.path.join(path, "adapter_model.bin"), map_location="cpu", weights_only=True)
        return cls.from_tensors(tensors, config)
