"""Fused-MoE activation quantisation to int8 through this package's kernels
(per-token dynamic / static per-tensor ``scaled_int8_quant``, per-group ``per_token_group_quant_int8``).
Parity: vllm_metax/patch/enhancement/utils.py:21-67."""
import torch

from .. import utils


@utils.patch("vllm.model_executor.layers.fused_moe.utils", "_int8_quantize")
def _int8_quantize(A: torch.Tensor, A_scale, per_act_token: bool, block_shape=None):
    from ... import _custom_ops as ops

    if block_shape is None:
        if per_act_token:
            q, s, _ = ops.scaled_int8_quant(A)
        else:
            if A_scale is None:
                A_scale = torch.clamp(A.abs().max().float() / 127.0, min=1e-10).reshape(1)
            q, s, _ = ops.scaled_int8_quant(A, scale=A_scale)
        return q, s
    assert not per_act_token and len(block_shape) == 2
    q, s = ops.per_token_group_quant_int8(A, block_shape[1])
    return q, s
