"""Registrations into upstream vLLM's extension points (only meaningful with vLLM installed):
``CustomOp.register_oot`` layers, linear kernels for the out-of-tree platform and quantisation configs.
Parity: vllm_metax/registry/__init__.py and its three sub-packages."""
try:
    import vllm  # noqa: F401

    HAVE_VLLM = True
except Exception:  # pragma: no cover
    HAVE_VLLM = False

if HAVE_VLLM:
    from . import custom_ops, fused_moe_method, linear_kernels, quant_config  # noqa: F401
