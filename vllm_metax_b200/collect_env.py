"""Environment report for bug reports: ``python -m vllm_metax_b200.collect_env`` (console script
``vllm_collect_env``).  Read-only: versions, GPUs / NVLink topology through NVML, CUDA toolchain, this
package's extension state and environment overrides.
Parity: vllm_metax/collect_env.py (env dump with driver / SDK / library versions)."""
from __future__ import annotations

import json
import os
import platform
import shutil
import subprocess
import sys


def _run(cmd: list[str]) -> str:
    try:
        return subprocess.run(cmd, capture_output=True, text=True, timeout=20).stdout.strip()
    except Exception as e:
        return f"<unavailable: {type(e).__name__}>"


def _version(mod: str) -> str:
    try:
        m = __import__(mod)
        return str(getattr(m, "__version__", "?"))
    except Exception:
        return "<not installed>"


def collect() -> dict:
    import torch

    from . import __version__, envs

    info: dict = {
        "package": {"vllm_metax_b200": __version__},
        "python": sys.version.replace("\n", " "),
        "os": platform.platform(),
        "libraries": {m: _version(m) for m in ("torch", "vllm", "transformers", "numpy", "triton", "flash_attn",
                                               "flashinfer", "pynvml")},
        "torch": {"cuda": torch.version.cuda, "cuda_available": torch.cuda.is_available(),
                  "nccl": ".".join(map(str, torch.cuda.nccl.version())) if torch.cuda.is_available() else None,
                  "arch_list": torch.cuda.get_arch_list() if torch.cuda.is_available() else []},
        "toolchain": {"nvcc": _run(["nvcc", "--version"]).splitlines()[-1:] if shutil.which("nvcc") else None,
                      "gcc": _run(["gcc", "--version"]).splitlines()[:1]},
    }
    try:
        from .utils import nvml

        with nvml.session() as n:
            info["gpus"] = n.summary()
            ids = list(range(n.device_count()))
            info["nvlink_fully_connected"] = n.fully_connected(ids) if len(ids) > 1 else None
    except Exception as e:
        info["gpus"] = f"<NVML unavailable: {e}>"
    try:
        from . import _build

        info["extension"] = {"library": str(_build.LIB), "built": _build.LIB.exists(),
                             "sources": len(_build.sources())}
    except Exception as e:
        info["extension"] = f"<{e}>"
    info["env"] = {k: v for k, v in sorted(os.environ.items())
                   if k.startswith(("B200_", "VLLM_", "NCCL_", "CUDA_", "TORCH_")) and "KEY" not in k and "TOKEN" not in k}
    info["overrides"] = {k: list(map(str, v)) for k, v in envs.overrides().items()}
    return info


def main() -> None:
    print(json.dumps(collect(), indent=2, default=str))


if __name__ == "__main__":
    main()
