"""vLLM out-of-tree platform for B200 (sm_100a): ``B200Platform``.

Returned (as a class path) by the ``vllm.platform_plugins`` entry point
``vllm_metax_b200:register``.  The platform presents itself to vLLM as an out-of-tree CUDA-like
device (``_enum = OOT``, ``device_type = "cuda"``, ``dispatch_key = "CUDA"``,
``dist_backend = "nccl"``) and routes vLLM's hook points to this package:

* ``get_attn_backend_cls``      -> the paged-GQA / MLA backends in ``vllm_metax_b200.vllm_backends``
* ``import_kernels``            -> loads ``_b200_C.so`` (``torch.ops.b200``)
* ``get_device_communicator_cls`` -> ``vllm_metax_b200.parallel.vllm_communicator.B200Communicator``
* ``check_and_update_config``   -> worker class, attention-op names, tuned-config folder
* device identity / topology queries through NVML (``utils/nvml.py``) with a torch fallback

Parity: vllm_metax/platform.py:76-1021 (MacaPlatformBase, the Mxsml / NonMxsml variants, the
backend priority lists :86-102, ``check_and_update_config`` :290-376, capability flags :562-697,
env overrides :994-1013).
"""
from __future__ import annotations

import os
from functools import lru_cache
from typing import TYPE_CHECKING, Any, Optional

import torch

from . import envs

try:  # vLLM is optional at import time (the standalone engine does not need it)
    from vllm.platforms.interface import DeviceCapability, Platform, PlatformEnum

    _HAVE_VLLM = True
except Exception:  # pragma: no cover - exercised only without vLLM
    _HAVE_VLLM = False

    class Platform:  # type: ignore
        pass

    class PlatformEnum:  # type: ignore
        OOT = "oot"

    class DeviceCapability(tuple):  # type: ignore
        def __new__(cls, major, minor):
            return super().__new__(cls, (major, minor))

if TYPE_CHECKING:
    from vllm.config import VllmConfig

# Attention backend name (vLLM's AttentionBackendEnum member) -> class path in this package.
# Dense decoder attention resolves to ONE backend whatever name the user picks among the GQA
# family; the MLA family likewise.
BACKEND_CLASS_PATHS = {
    "FLASH_ATTN": "vllm_metax_b200.vllm_backends.PagedGQABackend",
    "FLASH_ATTN_DIFFKV": "vllm_metax_b200.vllm_backends.PagedGQABackend",
    "FLASHINFER": "vllm_metax_b200.vllm_backends.PagedGQABackend",
    "TRITON_ATTN": "vllm_metax_b200.vllm_backends.PagedGQABackend",
    "FLASHMLA": "vllm_metax_b200.vllm_backends.MLABackend",
    "TRITON_MLA": "vllm_metax_b200.vllm_backends.MLABackend",
    "FLASHMLA_SPARSE": "vllm_metax_b200.vllm_backends.MLASparseBackend",
}
MLA_PRIORITY = ["FLASHMLA", "TRITON_MLA", "FLASHMLA_SPARSE"]
GQA_PRIORITY = ["FLASH_ATTN", "FLASHINFER", "TRITON_ATTN", "FLEX_ATTENTION"]


def _get_backend_priorities(use_mla: bool, use_sparse: bool = False) -> list[str]:
    if use_mla:
        return ["FLASHMLA_SPARSE"] if use_sparse else MLA_PRIORITY[:2]
    return list(GQA_PRIORITY)


def register_attention_backends() -> None:
    """Point vLLM's backend enum members at this package's classes."""
    from vllm.v1.attention.backends.registry import AttentionBackendEnum, register_backend

    for name, path in BACKEND_CLASS_PATHS.items():
        member = getattr(AttentionBackendEnum, name, None)
        if member is not None:
            register_backend(member, path)


class B200PlatformBase(Platform):
    _enum = PlatformEnum.OOT
    device_name: str = "b200"
    device_type: str = "cuda"
    dispatch_key: str = "CUDA"
    ray_device_key: str = "GPU"
    dist_backend: str = "nccl"
    device_control_env_var: str = "CUDA_VISIBLE_DEVICES"
    simple_compile_backend: str = "eager"

    supported_quantization: list[str] = [
        "awq", "auto_awq", "gptq", "auto_gptq", "compressed-tensors", "compressed_tensors", "moe_wna16", "gguf",
        "fp8", "deepseek_v4_fp8",
    ]

    # ------------------------------------------------------------------ device
    @classmethod
    def set_device(cls, device: torch.device) -> None:
        torch.cuda.set_device(device)
        torch.zeros(1, device=device)  # force context creation

    @classmethod
    def manual_seed_all(cls, seed: int) -> None:
        torch.cuda.manual_seed_all(seed)

    @classmethod
    def get_device_capability(cls, device_id: int = 0):
        if torch.cuda.is_available():
            major, minor = torch.cuda.get_device_capability(device_id)
            return DeviceCapability(major, minor)
        return DeviceCapability(10, 0)

    @classmethod
    def get_device_name(cls, device_id: int = 0) -> str:
        return torch.cuda.get_device_name(device_id) if torch.cuda.is_available() else "NVIDIA B200"

    @classmethod
    def get_device_total_memory(cls, device_id: int = 0) -> int:
        return torch.cuda.get_device_properties(device_id).total_memory

    @classmethod
    def get_device_uuid(cls, device_id: int = 0) -> str:
        return str(torch.cuda.get_device_properties(device_id).uuid)

    @classmethod
    def num_compute_units(cls, device_id: int = 0) -> int:
        return torch.cuda.get_device_properties(device_id).multi_processor_count

    @classmethod
    def is_fully_connected(cls, device_ids: list[int]) -> bool:
        return True  # NVSwitch: every pair of GPUs is one hop apart

    @classmethod
    def get_current_memory_usage(cls, device: Optional[torch.device] = None) -> float:
        torch.cuda.reset_peak_memory_stats(device)
        return torch.cuda.max_memory_allocated(device)

    @classmethod
    def is_integrated_gpu(cls, device_id: int = 0) -> bool:
        return False

    @classmethod
    def is_pin_memory_available(cls) -> bool:
        return True

    @classmethod
    def is_cuda_alike(cls) -> bool:
        return True

    def is_sleep_mode_available(self) -> bool:
        return True

    @classmethod
    def log_warnings(cls) -> None:
        pass

    # ------------------------------------------------------------------ kernels
    @classmethod
    def import_kernels(cls) -> None:
        from . import _custom_ops

        _custom_ops.load_native()
        # the kernel names upstream layers bind at construction time, on this package's kernels
        from .registry.c_namespace import define_c_ops

        define_c_ops()

    # ------------------------------------------------------------------ attention
    @classmethod
    def _late_registrations(cls) -> None:
        """Registrations that need upstream modules which cannot be imported while vLLM itself is still importing."""
        if _HAVE_VLLM:
            try:
                from .registry.fused_moe_method import ensure_registered

                ensure_registered()
            except Exception:  # registry layout differs between vLLM versions
                pass

    @classmethod
    def get_valid_backends(cls, attn_selector_config, device_capability=None) -> list[str]:
        use_mla = bool(getattr(attn_selector_config, "use_mla", False))
        use_sparse = bool(getattr(attn_selector_config, "use_sparse", False))
        return _get_backend_priorities(use_mla, use_sparse)

    @classmethod
    def get_attn_backend_cls(cls, selected_backend, attn_selector_config, num_heads: Optional[int] = None) -> str:
        cls._late_registrations()
        use_mla = bool(getattr(attn_selector_config, "use_mla", False))
        use_sparse = bool(getattr(attn_selector_config, "use_sparse", False))
        if selected_backend is not None:
            name = getattr(selected_backend, "name", str(selected_backend))
            if name in BACKEND_CLASS_PATHS:
                path = BACKEND_CLASS_PATHS[name]
                is_mla_backend = "MLA" in path
                if is_mla_backend != use_mla:
                    raise ValueError(f"backend {name} does not match use_mla={use_mla}")
                return path
            if name in ("FLEX_ATTENTION", "TORCH_SDPA"):
                return selected_backend.get_path() if hasattr(selected_backend, "get_path") else ""
            raise ValueError(f"attention backend {name} is not available on {cls.device_name}")
        return BACKEND_CLASS_PATHS[_get_backend_priorities(use_mla, use_sparse)[0]]

    @classmethod
    def get_supported_vit_attn_backends(cls):
        from vllm.v1.attention.backends.registry import AttentionBackendEnum

        return [AttentionBackendEnum.TORCH_SDPA]

    @classmethod
    def get_vit_attn_backend(cls, head_size: int, dtype: torch.dtype, backend=None):
        from vllm.v1.attention.backends.registry import AttentionBackendEnum

        return AttentionBackendEnum.TORCH_SDPA

    # ------------------------------------------------------------------ config hooks
    @classmethod
    def pre_register_and_update(cls, parser=None) -> None:
        if _HAVE_VLLM:
            try:
                register_attention_backends()
            except Exception:  # registry layout differs between vLLM versions
                pass

    @classmethod
    def check_and_update_config(cls, vllm_config: "VllmConfig") -> None:
        cls._late_registrations()
        parallel_config = vllm_config.parallel_config
        if getattr(parallel_config, "worker_cls", "auto") == "auto":
            parallel_config.worker_cls = "vllm.v1.worker.gpu_worker.Worker"
        cache_config = getattr(vllm_config, "cache_config", None)
        if cache_config is not None and getattr(cache_config, "block_size", None) is None:
            cache_config.block_size = 64
        model_config = getattr(vllm_config, "model_config", None)
        compilation = getattr(vllm_config, "compilation_config", None)
        if compilation is not None and _HAVE_VLLM:
            # This platform's hot path is hand-written kernels behind torch custom ops, not a tracing compiler:
            # the model runs as written (no Dynamo / Inductor pass) and decode steps are captured as whole CUDA
            # graphs, which the attention metadata builder supports for uniform decode batches.
            try:
                from vllm.config.compilation import CompilationMode, CUDAGraphMode

                enforce_eager = bool(getattr(model_config := getattr(vllm_config, "model_config", None),
                                             "enforce_eager", False))
                if getattr(compilation, "mode", None) not in (None, CompilationMode.NONE):
                    compilation.mode = CompilationMode.NONE
                if enforce_eager:
                    compilation.cudagraph_mode = CUDAGraphMode.NONE
                elif getattr(compilation, "cudagraph_mode", None) in (None, CUDAGraphMode.PIECEWISE,
                                                                      CUDAGraphMode.FULL_AND_PIECEWISE):
                    compilation.cudagraph_mode = CUDAGraphMode.FULL_DECODE_ONLY
            except ImportError:      # older config layout: leave vLLM's defaults
                pass
        if compilation is not None:
            ops_list = getattr(compilation, "_attention_ops", None)
            if isinstance(ops_list, list):
                for name in ("vllm::b200_sparse_attn_indexer", "vllm::b200_mla_attention"):
                    if name not in ops_list:
                        ops_list.append(name)
        if model_config is not None:
            # cascade attention is not implemented by the paged-GQA backend
            if hasattr(model_config, "disable_cascade_attn"):
                model_config.disable_cascade_attn = True
            hidden = getattr(getattr(model_config, "hf_text_config", None), "hidden_size", None)
            if hidden:
                folder = os.path.join(os.path.dirname(__file__), "layers", "moe_configs", f"H={hidden}")
                if os.path.isdir(folder):
                    envs.override_env("VLLM_TUNED_CONFIG_FOLDER", folder, "tuned MoE tiles for this hidden size",
                                      forward_to_vllm=True)

    # ------------------------------------------------------------------ capability flags
    @classmethod
    def get_device_communicator_cls(cls) -> str:
        return "vllm_metax_b200.parallel.vllm_communicator.B200Communicator"

    @classmethod
    def supports_fp8(cls) -> bool:
        return bool(envs.B200_SUPPORTS_FP8)

    @classmethod
    def use_custom_allreduce(cls) -> bool:
        return False  # the fused row-parallel kernels own the all-reduce

    @classmethod
    def opaque_attention_op(cls) -> bool:
        return True

    @classmethod
    def get_static_graph_wrapper_cls(cls) -> str:
        return "vllm.compilation.cuda_graph.CUDAGraphWrapper"

    @classmethod
    def support_hybrid_kv_cache(cls) -> bool:
        return True

    @classmethod
    def support_static_graph_mode(cls) -> bool:
        return True

    @classmethod
    def support_deep_gemm(cls) -> bool:
        return False  # block-scaled fp8 GEMMs are this package's own kernels

    @classmethod
    def use_custom_op_collectives(cls) -> bool:
        return True

    @classmethod
    def get_default_ir_op_priority(cls, vllm_config):
        """Kernel-provider order for vLLM's IR ops: this package's CUDA ops (registered under the ``vllm_c``
        provider name through the custom-op registry) first, the native PyTorch lowering as the fall-back
        (vllm_metax/platform.py:666-688)."""
        from vllm.config.kernel import IrOpPriorityConfig

        default = ["vllm_c", "native"]
        return IrOpPriorityConfig.with_default(default, rms_norm=default, fused_add_rms_norm=default)

    @classmethod
    def get_punica_wrapper(cls) -> str:
        return "vllm.lora.punica_wrapper.punica_gpu.PunicaWrapperGPU"

    @classmethod
    def check_if_supports_dtype(cls, dtype: torch.dtype) -> None:
        if dtype not in (torch.bfloat16, torch.float16, torch.float32):
            raise ValueError(f"{dtype} is not supported on {cls.device_name}")

    @classmethod
    def stateless_init_device_torch_dist_pg(cls, backend: str, prefix_store, group_rank: int, group_size: int,
                                            timeout):
        from torch.distributed import ProcessGroup
        from torch.distributed.distributed_c10d import ProcessGroupNCCL

        pg = ProcessGroup(prefix_store, group_rank, group_size)
        opts = ProcessGroupNCCL.Options()
        opts._timeout = timeout
        backend_cls = ProcessGroupNCCL(prefix_store, group_rank, group_size, opts)
        backend_type = ProcessGroup.BackendType.NCCL
        device = torch.device("cuda")
        pg._set_default_backend(backend_type)
        backend_cls._set_sequence_number_for_group()
        pg._register_backend(device, backend_type, backend_cls)
        return pg

    @classmethod
    def insert_blocks_to_device(cls, src_cache, dst_cache, src_block_indices, dst_block_indices) -> None:
        dst_cache[:, dst_block_indices] = src_cache[:, src_block_indices].to(dst_cache.device)

    @classmethod
    def swap_out_blocks_to_host(cls, src_cache, dst_cache, src_block_indices, dst_block_indices) -> None:
        dst_cache[:, dst_block_indices] = src_cache[:, src_block_indices].cpu()


class NvmlB200Platform(B200PlatformBase):
    """Identity and topology through NVML (handles CUDA_VISIBLE_DEVICES remapping, no CUDA context)."""

    @classmethod
    def _nvml(cls):
        from .utils import nvml

        return nvml

    @classmethod
    def _physical(cls, device_id: int) -> int:
        vis = os.environ.get(cls.device_control_env_var)
        if vis:
            ids = [x for x in vis.split(",") if x != ""]
            try:
                return int(ids[device_id])
            except (ValueError, IndexError):
                return device_id
        return device_id

    @classmethod
    @lru_cache(maxsize=8)
    def get_device_capability(cls, device_id: int = 0):
        with cls._nvml().session() as n:
            major, minor = n.device_capability(cls._physical(device_id))
        return DeviceCapability(major, minor)

    @classmethod
    def get_device_name(cls, device_id: int = 0) -> str:
        with cls._nvml().session() as n:
            return n.device_name(cls._physical(device_id))

    @classmethod
    def get_device_uuid(cls, device_id: int = 0) -> str:
        with cls._nvml().session() as n:
            return n.device_uuid(cls._physical(device_id))

    @classmethod
    def get_device_total_memory(cls, device_id: int = 0) -> int:
        with cls._nvml().session() as n:
            return n.device_memory_total(cls._physical(device_id))

    @classmethod
    def is_fully_connected(cls, device_ids: list[int]) -> bool:
        with cls._nvml().session() as n:
            return n.fully_connected([cls._physical(i) for i in device_ids])

    @classmethod
    def get_device_numa_node(cls, device_id: int = 0) -> Optional[int]:
        with cls._nvml().session() as n:
            return n.device_numa_node(cls._physical(device_id))

    @classmethod
    def get_all_device_numa_nodes(cls) -> list[Optional[int]]:
        with cls._nvml().session() as n:
            return [n.device_numa_node(i) for i in range(n.device_count())]

    @classmethod
    def get_all_gpu_pci_bus_ids(cls) -> list[str]:
        with cls._nvml().session() as n:
            return [n.device_pci_bus_id(i) for i in range(n.device_count())]


class TorchB200Platform(B200PlatformBase):
    """Fallback when NVML is unavailable: everything through torch.cuda."""


def _autodetect():
    try:
        from .utils import nvml

        with nvml.session() as n:
            n.device_count()
        return NvmlB200Platform
    except Exception:
        return TorchB200Platform


B200Platform = _autodetect()

# Runtime defaults this platform wants from vLLM (applied on import, as the plugin loader imports
# this module in every process).
if _HAVE_VLLM:
    for _name, _val, _why in (
        # typed as vllm.envs returns them (the override replaces vLLM's parser for the name)
        ("VLLM_USE_FLASHINFER_SAMPLER", False, "sampling runs on this package's kernels"),
        ("VLLM_ENGINE_READY_TIMEOUT_S", 7200, "first start compiles / captures graphs"),
        ("VLLM_FLOAT32_MATMUL_PRECISION", "high", "fp32 matmuls may use tf32"),
    ):
        if _name not in os.environ:
            envs.override_env(_name, _val, _why, forward_to_vllm=True)
