"""Tuned fused-MoE launch parameters, looked up by problem shape.

A config file is named ``E=<experts>,N=<intermediate per rank>,device_name=<gpu>[,dtype=<w4a16|fp8_w8a8|int8_w8a8>].json``
under ``H=<hidden>/`` and maps a token count M to launch parameters ``{"token_tile": ...}`` (the row-block size that
``moe_align_block_size`` pads each expert to; 128 for the bf16 / fp8 / int8 grouped tcgen05 GEMMs, 16..128 for the
weight-only kernel) - optionally split per GEMM as ``{"stage1": {...}, "stage2": {...}}``.  The nearest M not above
the batch's token count is used.  ``VLLM_TUNED_CONFIG_FOLDER`` (set by the platform's ``check_and_update_config``)
points at the folder for the model's hidden size; user folders work the same way.
Parity: vllm_metax/model_executor/layers/fused_moe/fused_moe.py:1331-1409 (get_moe_configs, H-prefixed lookup),
:1536-1633 (get_default_config), :1636-1679 (two-stage configs), configs/H=*/ tuned JSON files.
"""
from __future__ import annotations

import functools
import json
import os
from typing import Optional

HERE = os.path.dirname(os.path.abspath(__file__))


def config_file_name(E: int, N: int, device_name: str, dtype: Optional[str] = None) -> str:
    dev = device_name.replace(" ", "_")
    return f"E={E},N={N},device_name={dev}" + (f",dtype={dtype}" if dtype else "") + ".json"


@functools.lru_cache(maxsize=64)
def get_moe_configs(E: int, N: int, hidden: int, device_name: str = "NVIDIA_B200", dtype: Optional[str] = None):
    """{M: config} from the first folder that has the file: $VLLM_TUNED_CONFIG_FOLDER, then the packaged H=<hidden>/."""
    name = config_file_name(E, N, device_name, dtype)
    folders = [f for f in (os.environ.get("VLLM_TUNED_CONFIG_FOLDER"), os.path.join(HERE, f"H={hidden}")) if f]
    for folder in folders:
        path = os.path.join(folder, name)
        if os.path.isfile(path):
            with open(path) as f:
                return {int(k): v for k, v in json.load(f).items()}
    return None


def get_default_config(M: int, E: int, topk: int, dtype: Optional[str] = None) -> dict:
    """Heuristic when no tuned file exists: small per-expert batches use small token tiles on the weight-only path."""
    if dtype == "w4a16":
        per_expert = max(1, M * topk // max(E, 1))
        tile = 16 if per_expert <= 16 else 32 if per_expert <= 32 else 64 if per_expert <= 64 else 128
    else:
        tile = 128
    return {"token_tile": tile}


def try_get_optimal_moe_config(M: int, E: int, N: int, hidden: int, topk: int, dtype: Optional[str] = None,
                               device_name: str = "NVIDIA_B200") -> dict:
    cfgs = get_moe_configs(E, N, hidden, device_name, dtype)
    if not cfgs:
        return get_default_config(M, E, topk, dtype)
    keys = sorted(cfgs)
    best = keys[0]
    for k in keys:
        if k <= M:
            best = k
    return cfgs[best]


def stage_config(cfg: dict, stage: int) -> dict:
    """Two-stage files carry separate parameters for the w13 and w2 GEMMs."""
    key = f"stage{stage}"
    return cfg[key] if key in cfg else cfg
