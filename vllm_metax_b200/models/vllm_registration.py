"""``vllm.general_plugins`` entry point ``register_model``: offer this package's model classes to vLLM's
``ModelRegistry`` under the architecture names of the checkpoints (lazy ``module:Class`` strings, so
nothing is imported until vLLM resolves an architecture).
Parity: vllm_metax/models/__init__.py:6-38."""
from __future__ import annotations

from . import _MODELS

# architectures this package overrides when running under vLLM (the dense / MoE families are served by
# upstream model code + this platform's kernels, as in the reference)
VLLM_ARCHITECTURES = (
    "DeepseekV2ForCausalLM", "DeepseekV3ForCausalLM", "DeepseekV32ForCausalLM", "GlmMoeDsaForCausalLM",
    "DeepSeekMTPModel", "DeepseekV4ForCausalLM", "DeepSeekV4MTPModel", "Step3p5MTP",
)


def register_with_vllm(architectures=VLLM_ARCHITECTURES) -> list[str]:
    try:
        from vllm import ModelRegistry
    except Exception:
        return []
    done = []
    for arch in architectures:
        if arch not in _MODELS:
            continue
        mod, cls = _MODELS[arch]
        ModelRegistry.register_model(arch, f"{__package__}.{mod}:{cls}")
        done.append(arch)
    return done
