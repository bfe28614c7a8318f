"""Unquantised ``FusedMoE`` experts of upstream vLLM on this package's grouped tcgen05 GEMMs.

Upstream picks the expert kernel through ``select_unquantized_moe_backend``; on an out-of-tree platform that answers
``OOT`` ("the platform handles it") and sets up no kernel, so the method registered here does the work: at load time
the gate / up halves of ``w13`` are interleaved row by row (the layout whose SiLU-gate the grouped GEMM applies in its
epilogue), at run time the routed pairs go through align -> gather -> grouped GEMM (+ SiLU-gate) -> grouped GEMM ->
weighted combine (``layers/fused_moe.py:fused_experts``).  Shared experts are applied through upstream's hook.
Parity: vllm_metax/registry/custom_ops/layers/fused_moe/unquantized_fused_moe_method.py:37-103 (same registration
name, Triton experts there).
"""
from __future__ import annotations

import torch

from ..layers.fused_moe import fused_experts

REGISTERED = False
_CLASS = None


def interleave_gate_up(w13: torch.Tensor) -> torch.Tensor:
    """``[E, 2I, H]`` with rows (gate_0..gate_{I-1}, up_0..up_{I-1}) -> rows (gate_0, up_0, gate_1, up_1, ...)."""
    E, two_i, H = w13.shape
    half = two_i // 2
    return torch.stack([w13[:, :half], w13[:, half:]], dim=2).reshape(E, two_i, H)


def _build_class():
    from vllm.model_executor.layers.fused_moe.unquantized_fused_moe_method import (
        UnquantizedFusedMoEMethod as _Upstream)

    class B200UnquantizedFusedMoEMethod(_Upstream):
        """Registered under upstream's name, so every unquantised ``FusedMoE`` layer is built with it."""

        @property
        def is_monolithic(self) -> bool:
            return False        # routing stays with upstream's router; this method is handed (weights, ids)

        def process_weights_after_loading(self, layer: torch.nn.Module) -> None:
            super().process_weights_after_loading(layer)
            # (also after a weight update: the loader rewrites w13 in checkpoint order, in place)
            w13 = layer.w13_weight.data
            layer.w13_weight.data.copy_(interleave_gate_up(w13))     # same storage: captured graphs stay valid
            layer._b200_interleaved = True

        def forward_oot(self, layer, x, topk_weights, topk_ids, shared_experts=None, shared_experts_input=None):
            act = getattr(layer, "activation", None)
            act_name = str(getattr(act, "value", act)).lower()
            if ("silu" not in act_name or getattr(layer, "apply_router_weight_on_input", False)
                    or getattr(layer, "w13_bias", None) is not None):
                raise NotImplementedError(f"unquantised experts on this platform: SiLU-gated, no bias (got {act_name})")
            x2 = x.reshape(-1, x.shape[-1])
            out = fused_experts(x2, layer.w13_weight, layer.w2_weight, topk_weights.float().contiguous(),
                                topk_ids.to(torch.int32).contiguous(), layer.w13_weight.shape[0],
                                getattr(layer, "expert_map", None))
            if shared_experts is not None:
                from vllm.model_executor.layers.fused_moe.modular_kernel import SharedExpertsOrder

                shared_experts.apply(shared_experts_input if shared_experts_input is not None else x,
                                     SharedExpertsOrder.MK_INTERNAL_OVERLAPPED)
            return out.reshape(x.shape)

    return _Upstream, B200UnquantizedFusedMoEMethod


def ensure_registered() -> bool:
    """Registers the method once upstream's MoE modules can be imported.  The general-plugin hook may run in the
    middle of vLLM's own imports (a circular import then), so the platform calls this again when it is asked for an
    attention backend - which happens before the first MoE layer of a model is built, in every process."""
    global REGISTERED, _CLASS
    if REGISTERED:
        return True
    try:
        upstream, cls = _build_class()
    except Exception:
        return False
    try:
        upstream.register_oot(cls, name="UnquantizedFusedMoEMethod")
    except AssertionError:      # another plugin registered the name first
        return False
    _CLASS = cls
    REGISTERED = True
    return True


ensure_registered()
