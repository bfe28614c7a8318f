"""vllm_metax_b200 - a Blackwell (sm_100a) native serving framework with the capability
surface of the vLLM-metax platform plugin.

Two ways in:

* standalone: ``from vllm_metax_b200 import LLM, SamplingParams`` (own engine, scheduler,
  paged KV cache, OpenAI-compatible server in ``entrypoints``);
* as a vLLM out-of-tree platform plugin through the three entry points below
  (``vllm.platform_plugins`` / ``vllm.general_plugins``), mirroring
  vllm_metax/__init__.py:7-38.
"""
import logging as _logging
import os as _os

from .version import __version__  # noqa: F401

# B200_LOG_LEVEL: level of the package's loggers (DEBUG / INFO / WARNING / ...)
_logging.getLogger(__name__).setLevel(getattr(_logging, _os.environ.get("B200_LOG_LEVEL", "INFO").upper(), _logging.INFO))


if _os.environ.get("B200_BATCH_INVARIANT", "0") not in ("", "0"):
    from . import _custom_ops as _ops      # pins the dependent switches before anything reads them

    _ops.batch_invariant()


def collect_env() -> None:
    from .collect_env import main

    main()


def register() -> str:
    """``vllm.platform_plugins`` entry point: class path of the Platform subclass."""
    return "vllm_metax_b200.platform.B200Platform"


def _patch() -> None:
    from . import patch  # noqa: F401  (each @patch applies on import)


def _out_of_tree() -> None:
    from . import registry  # noqa: F401


def register_out_of_tree() -> None:
    """``vllm.general_plugins`` entry point: apply patches, then the op / quant registries."""
    _patch()
    _out_of_tree()


def register_model() -> None:
    """``vllm.general_plugins`` entry point: register model architectures with vLLM."""
    from .models.vllm_registration import register_with_vllm

    register_with_vllm()


def __getattr__(name):
    if name in ("LLM", "LLMEngine", "EngineDeadError"):
        from .engine import llm

        return getattr(llm, name)
    if name in ("SamplingParams", "RequestOutput"):
        from .engine import sampling_params

        return getattr(sampling_params, name)
    if name == "ModelConfig":
        from .config import ModelConfig

        return ModelConfig
    raise AttributeError(name)
