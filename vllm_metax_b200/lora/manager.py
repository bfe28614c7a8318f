"""Adapter slots on the model's linears and the per-batch routing of rows to adapters."""
from __future__ import annotations

from collections import OrderedDict
from typing import Optional

import torch
import torch.nn as nn

from ..layers.linear import RowParallelLinear
from ..parallel import state as ps
from .models import LoRAModel
from .request import LoRARequest

# fused module name -> ordered shard ids (each takes `rank` columns of the stacked rank dimension)
SHARDS = {"qkv_proj": ("q", "k", "v"), "gate_up_proj": (0, 1), "o_proj": (None,), "down_proj": (None,)}


class _ModuleState:
    def __init__(self, module: nn.Module, kind: str, max_loras: int, max_rank: int, device, dtype):
        self.module, self.kind = module, kind
        self.shards = SHARDS[kind]
        w = module.weight
        self.out_local, self.in_local = w.shape[0], w.shape[1]
        R = max_rank * len(self.shards)
        self.A = torch.zeros(max_loras, R, self.in_local, dtype=dtype, device=device)
        self.B = torch.zeros(max_loras, self.out_local, R, dtype=dtype, device=device)
        self.max_rank = max_rank
        self.row_parallel = isinstance(module, RowParallelLinear)

    def clear(self, slot: int) -> None:
        self.A[slot].zero_()
        self.B[slot].zero_()

    def load(self, slot: int, parts: dict, rank: int) -> None:
        """``parts``: shard id -> (A [r, in_full], B [out_full, r]) in fp32 on CPU."""
        self.clear(slot)
        m, r0 = self.module, self.max_rank
        for i, sid in enumerate(self.shards):
            if sid not in parts:
                continue
            a, b = parts[sid]
            a_dst = torch.zeros(rank, self.in_local)
            if self.row_parallel:
                m.weight_loader(a_dst, a)                       # input dimension sharded like the base weight
                b_dst = b                                        # output replicated
            else:
                a_dst = a                                        # input replicated
                b_dst = torch.zeros(self.out_local, rank)
                m.weight_loader(b_dst, b, sid)                  # output rows cut and placed like the base weight
            self.A[slot, i * r0: i * r0 + rank].copy_(a_dst)
            self.B[slot, :, i * r0: i * r0 + rank].copy_(b_dst)


class LoRAManager:
    def __init__(self, model: nn.Module, max_loras: int, max_rank: int, device, dtype):
        self.max_loras, self.max_rank = max_loras, max_rank
        self.device, self.dtype = device, dtype
        self.states: dict[str, _ModuleState] = {}
        for name, mod in model.named_modules():
            kind = name.rsplit(".", 1)[-1]
            if kind in SHARDS and hasattr(mod, "weight") and mod.weight.dim() == 2 and hasattr(mod, "weight_loader"):
                if type(mod).__name__ == "GateUpSiluLinear":
                    raise RuntimeError("gate_up_proj has its activation fused; build the model with enable_lora=True")
                st = _ModuleState(mod, kind, max_loras, max_rank, device, dtype)
                self.states[name] = st
                mod.register_forward_hook(self._make_hook(st))
        if not self.states:
            raise RuntimeError("no LoRA target modules found in the model")
        self.slot_of: "OrderedDict[int, int]" = OrderedDict()      # lora_int_id -> slot, least recently used first
        self.scaling = torch.zeros(max_loras, dtype=torch.float32)
        self.batch_slots: Optional[torch.Tensor] = None             # int64 [T] slot per row, -1 = base model
        self.batch_active: list[int] = []
        self.tp_group = ps.get_tp_group() if ps.tp_size() > 1 else None

    # ------------------------------------------------------------------ adapters
    def activate(self, req: LoRARequest, in_use: Optional[set] = None) -> int:
        """Slot of the adapter, loading it (and evicting the least recently used idle one) when needed."""
        lid = req.lora_int_id
        if lid in self.slot_of:
            self.slot_of.move_to_end(lid)
            return self.slot_of[lid]
        if len(self.slot_of) < self.max_loras:
            slot = next(s for s in range(self.max_loras) if s not in self.slot_of.values())
        else:
            victim = next((k for k in self.slot_of if in_use is None or k not in in_use), None)
            if victim is None:
                raise RuntimeError(f"more than max_loras={self.max_loras} adapters are needed by one batch")
            slot = self.slot_of.pop(victim)
        lm = (LoRAModel.from_tensors(req.tensors, req.config) if req.tensors is not None
              else LoRAModel.from_peft_dir(req.lora_path))
        if lm.rank > self.max_rank:
            raise ValueError(f"adapter rank {lm.rank} exceeds max_lora_rank={self.max_rank}")
        seen = set()
        for (mod, fused), parts in lm.weights.items():
            st = self.states.get(f"{mod}.{fused}")
            if st is None:
                raise ValueError(f"adapter targets {mod}.{fused}, which this model does not have")
            st.load(slot, parts, lm.rank)
            seen.add(f"{mod}.{fused}")
        for name, st in self.states.items():
            if name not in seen:
                st.clear(slot)
        self.scaling[slot] = lm.scaling
        self.slot_of[lid] = slot
        return slot

    def remove(self, lora_int_id: int) -> bool:
        return self.slot_of.pop(lora_int_id, None) is not None

    def list_adapters(self) -> list[int]:
        return list(self.slot_of)

    # ------------------------------------------------------------------ batches
    def set_batch(self, row_slots: Optional[list]) -> None:
        """``row_slots``: slot per row of the step's token batch (-1 = no adapter), or None."""
        if row_slots is None or all(s < 0 for s in row_slots):
            self.batch_slots, self.batch_active = None, []
            return
        self.batch_slots = torch.tensor(row_slots, dtype=torch.long, device=self.device)
        self.batch_active = sorted({s for s in row_slots if s >= 0})

    def _make_hook(self, st: _ModuleState):
        def hook(module, inputs, output):
            if self.batch_slots is None:
                return output
            x = inputs[0]
            x2 = x.reshape(-1, x.shape[-1])
            y2 = output.reshape(-1, output.shape[-1])
            T = x2.shape[0]
            slots = self.batch_slots[:T]
            for s in self.batch_active:
                idx = (slots == s).nonzero(as_tuple=True)[0]
                if idx.numel() == 0:
                    continue
                xa = x2.index_select(0, idx) @ st.A[s].t()                   # shrink: [n, R]
                if st.row_parallel and self.tp_group is not None:
                    xa = self.tp_group.all_reduce(xa.float()).to(x2.dtype)   # partial sums over the input shards
                delta = (xa @ st.B[s].t()) * float(self.scaling[s])          # expand: [n, out_local]
                y2.index_add_(0, idx, delta.to(y2.dtype))
            return output

        return hook
