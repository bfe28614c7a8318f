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


def register_with_vllm(architectures=VLLM_ARCHITECTURES, force: bool = False) -> list[str]:
    """Registers the classes that declare ``vllm_compatible = True`` (constructor ``(vllm_config, prefix)`` and
    vLLM's attention layers inside).  The standalone classes of this package take a ``ModelConfig`` and run on the
    package's own attention metadata, so they are NOT offered to vLLM: under vLLM those architectures run upstream's
    model code on this platform's kernels and backends.  ``force`` registers regardless (tests of the plumbing)."""
    try:
        from vllm import ModelRegistry
    except Exception:
        return []
    import importlib

    done = []
    for arch in architectures:
        if arch not in _MODELS:
            continue
        mod, cls = _MODELS[arch]
        if not force:
            try:
                klass = getattr(importlib.import_module(f"{__package__}.{mod}"), cls)
            except Exception:
                continue
            if not getattr(klass, "vllm_compatible", False):
                continue
        ModelRegistry.register_model(arch, f"{__package__}.{mod}:{cls}")
        done.append(arch)
    return done
