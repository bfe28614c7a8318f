"""Make the block-scaled fp8 linear kernel of this package the choice for the out-of-tree platform.
Parity: vllm_metax/patch/enhancement/quant_kernels/fp8_block_kernel.py:8-20."""
try:
    from vllm.model_executor.kernels import linear as _linear
    from vllm.platforms import PlatformEnum

    from ...registry.linear_kernels import B200Fp8BlockScaledMMKernel

    table = getattr(_linear, "_POSSIBLE_FP8_BLOCK_KERNELS", None)
    if isinstance(table, dict):
        table[PlatformEnum.OOT] = [B200Fp8BlockScaledMMKernel]
except Exception:  # upstream layout differs or vLLM missing: nothing to do
    pass
