"""Grouped top-k routing (DeepSeek-V2/V3 style) through ONE kernel launch.

``GroupedTopKRouter._compute_routing`` is replaced so that score (softmax / sigmoid / sqrt-softplus),
correction bias, group selection, expert top-k, renormalisation and the routed scaling factor all
run in ``ops.grouped_topk`` (one warp per token).  Shapes the kernel does not cover (more than 512
experts, more than 32 groups or top-k above 32) fall back to the upstream implementation.
Parity: vllm_metax/patch/performance/grouped_topk_router.py:40-284.
"""
import torch

from .. import utils

_upstream = None


def kernel_covers(num_experts: int, num_expert_group: int, topk_group: int, top_k: int) -> bool:
    if num_expert_group <= 0 or num_experts % num_expert_group:
        return False
    return num_experts <= 512 and num_expert_group <= 32 and top_k <= 32 and topk_group <= num_expert_group


def b200_grouped_topk(gating_output: torch.Tensor, topk: int, renormalize: bool, num_expert_group: int,
                      topk_group: int, scoring_func: str = "softmax", routed_scaling_factor: float = 1.0,
                      e_score_correction_bias: torch.Tensor | None = None,
                      indices_type: torch.dtype | None = None):
    from ... import _custom_ops as ops

    w, ids = ops.grouped_topk(gating_output, topk, renormalize, num_expert_group, topk_group,
                              scoring_func=scoring_func, bias=e_score_correction_bias,
                              routed_scaling_factor=routed_scaling_factor)
    if indices_type is not None and ids.dtype != indices_type:
        ids = ids.to(indices_type)
    return w, ids


def _compute_routing(self, hidden_states, router_logits, indices_type, *, input_ids=None):
    E = router_logits.shape[-1]
    if (router_logits.is_cuda and self.scoring_func in ("softmax", "sigmoid") and getattr(self, "num_fused_shared_experts", 0) == 0
            and E > self.num_expert_group and kernel_covers(E, self.num_expert_group, self.topk_group, self.top_k)):
        return b200_grouped_topk(router_logits, self.top_k, self.renormalize, self.num_expert_group, self.topk_group,
                                 self.scoring_func, self.routed_scaling_factor, self.e_score_correction_bias,
                                 indices_type)
    return _upstream(self, hidden_states, router_logits, indices_type, input_ids=input_ids)


try:
    from vllm.model_executor.layers.fused_moe.router import grouped_topk_router as _mod

    _upstream = _mod.GroupedTopKRouter._compute_routing
    utils.apply_patch("vllm.model_executor.layers.fused_moe.router.grouped_topk_router",
                      "GroupedTopKRouter._compute_routing", _compute_routing)
except ImportError:
    pass
