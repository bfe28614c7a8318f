"""Model construction and weight loading.

Formats: ``dummy`` (seeded normal(0, 0.02) init of every parameter - what benchmarks and
tests use), HF ``safetensors`` shards (single file or ``model.safetensors.index.json``),
and ``sharded_state`` (one ``rank{r}.safetensors`` per TP rank holding already-sharded
parameters, saved by ``save_sharded_state``).  Quantised checkpoints keep their on-disk
tensor names (``weight``, ``weight_scale_inv``, ``qweight`` ...); each layer's quant
method owns the parameter layout and any post-load repacking.

Parity: the reference takes all of this from upstream loaders and adds per-format repacking
at load (vllm_metax/registry/quant_config/auto_awq.py:74-85, fp8.py:101-117,
models/deepseek_v2.py:1496-1733).
"""
from __future__ import annotations

import glob
import json
import os
from typing import Iterator

import torch
import torch.nn as nn

from ..config import EngineConfig
from ..models import get_model_class


def build_model(cfg: EngineConfig, device: torch.device) -> nn.Module:
    cls = get_model_class(cfg.model.architecture)
    prev = torch.get_default_dtype()
    with torch.device(device):
        model = cls(cfg.model)
    torch.set_default_dtype(prev)
    fmt = cfg.load_format
    if fmt == "auto":
        fmt = "safetensors" if cfg.model.model_path else "dummy"
    if fmt == "dummy":
        dummy_init(model, cfg.model.seed)
        for m in model.modules():
            qm = getattr(m, "quant_method", None)
            if qm is not None and hasattr(qm, "process_weights_after_loading"):
                qm.process_weights_after_loading(m)
        if hasattr(model, "finalize_weights"):
            model.finalize_weights()
    elif fmt == "safetensors":
        model.load_weights(iter_safetensors(cfg.model.model_path))
    elif fmt == "sharded_state":
        load_sharded_state(model, cfg.model.model_path)
    else:
        raise ValueError(f"unknown load_format {fmt}")
    return model.eval()


@torch.no_grad()
def dummy_init(model: nn.Module, seed: int = 0, std: float = 0.02) -> None:
    """Seeded init generated on the parameter's own device (fast for multi-billion-parameter
    models).  Values differ between CPU and GPU generators; tests that compare devices copy a
    state dict instead."""
    for name, p in model.named_parameters():
        g = torch.Generator(device=p.device)
        g.manual_seed((seed * 1000003 + (hash_name(name) % 1000003)) % (2 ** 31))
        if p.dtype in (torch.float32, torch.bfloat16, torch.float16):
            if name.endswith("norm.weight") or name.endswith("layernorm.weight") or ".norm." in name and p.dim() == 1:
                p.data.fill_(1.0)
                continue
            if getattr(p, "is_scale", False):
                p.data.copy_(torch.rand(p.shape, generator=g, device=p.device).mul_(0.02).add_(0.005).to(p.dtype))
                continue
            w = torch.empty(p.shape, dtype=torch.float32, device=p.device).normal_(0.0, std, generator=g)
            p.data.copy_(w.to(p.dtype))
        elif p.dtype == torch.float8_e4m3fn:
            w = torch.empty(p.shape, dtype=torch.float32, device=p.device).normal_(0.0, 1.0, generator=g)
            p.data.copy_(w.clamp(-448, 448).to(torch.float8_e4m3fn))
        elif p.dtype == torch.int8:
            p.data.copy_(torch.randint(-127, 128, p.shape, generator=g, dtype=torch.int32, device=p.device).to(torch.int8))
        elif p.dtype == torch.int32:
            p.data.copy_(torch.randint(-2 ** 31, 2 ** 31 - 1, p.shape, generator=g, dtype=torch.int64, device=p.device).to(torch.int32))


def hash_name(name: str) -> int:
    h = 1469598103934665603
    for ch in name.encode():
        h = ((h ^ ch) * 1099511628211) & 0xFFFFFFFFFFFFFFFF
    return h


def iter_safetensors(path: str) -> Iterator[tuple[str, torch.Tensor]]:
    if path.endswith(".gguf"):
        from .gguf import iter_gguf

        yield from iter_gguf(path, torch.float32)       # parameters cast on copy
        return
    from safetensors import safe_open

    index = os.path.join(path, "model.safetensors.index.json")
    if os.path.exists(index):
        with open(index) as f:
            files = sorted(set(json.load(f)["weight_map"].values()))
        files = [os.path.join(path, x) for x in files]
    else:
        files = sorted(glob.glob(os.path.join(path, "*.safetensors")))
    if not files:
        raise FileNotFoundError(f"no safetensors files under {path}")
    for fn in files:
        with safe_open(fn, framework="pt", device="cpu") as f:
            for k in f.keys():
                yield k, f.get_tensor(k)


def save_sharded_state(model: nn.Module, path: str, rank: int) -> None:
    from safetensors.torch import save_file

    os.makedirs(path, exist_ok=True)
    sd = {k: v.detach().cpu().contiguous() for k, v in model.named_parameters()}
    for k, v in list(sd.items()):
        if v.dtype == torch.float8_e4m3fn:
            sd[k] = v.view(torch.uint8)
            sd[k + ".__fp8__"] = torch.zeros(1, dtype=torch.uint8)
    save_file(sd, os.path.join(path, f"rank{rank}.safetensors"))


def load_sharded_state(model: nn.Module, path: str) -> None:
    from safetensors.torch import load_file

    from ..parallel import state as ps

    sd = load_file(os.path.join(path, f"rank{ps.global_rank()}.safetensors"))
    params = dict(model.named_parameters())
    for k, v in sd.items():
        if k.endswith(".__fp8__"):
            continue
        if k + ".__fp8__" in sd:
            v = v.view(torch.float8_e4m3fn)
        params[k].data.copy_(v)
