r"""Per-module precision dump: forward hooks that record summary statistics (shape, dtype, mean, abs-max, L2 norm,
NaN / Inf counts and a position-weighted checksum) of every module output to a JSONL file, and a comparer that
lines two dumps up (e.g. CPU fp32 vs GPU bf16, or two kernel versions) and reports the first divergence.

    with PrecisionDump(model, "gpu.jsonl", pattern=r"layers\.\d+\.(self_attn|mlp)$"):
        llm.generate(...)
    print(compare_dumps("cpu.jsonl", "gpu.jsonl", rtol=5e-2))

Parity: the reference's precision-debugging guide (docs/developing/msprobe/msprobe_guide.md: dump per-layer
tensors on both platforms, compare, locate the first bad module).
"""
from __future__ import annotations

import json
import re
from typing import Optional

import torch
import torch.nn as nn


def tensor_stats(t: torch.Tensor) -> dict:
    f = t.detach().float().reshape(-1)
    n = f.numel()
    if n == 0:
        return {"shape": list(t.shape), "dtype": str(t.dtype), "numel": 0}
    finite = torch.isfinite(f)
    g = torch.where(finite, f, torch.zeros_like(f))
    w = (torch.arange(n, device=f.device, dtype=torch.float32) % 97 + 1.0) / 97.0
    return {"shape": list(t.shape), "dtype": str(t.dtype), "numel": n, "mean": float(g.mean()),
            "absmax": float(g.abs().max()), "l2": float(g.norm()), "nan": int(torch.isnan(f).sum()),
            "inf": int(torch.isinf(f).sum()), "checksum": float((g * w).sum())}


class PrecisionDump:
    def __init__(self, model: nn.Module, path: str, pattern: Optional[str] = None, max_records: int = 100000):
        self.model, self.path = model, path
        self.pattern = re.compile(pattern) if pattern else None
        self.max_records = max_records
        self._handles: list = []
        self._calls: dict[str, int] = {}
        self._fh = None
        self._n = 0

    def _hook(self, name: str):
        def fn(_mod, _inp, out):
            if self._n >= self.max_records:
                return
            outs = out if isinstance(out, (tuple, list)) else (out,)
            call = self._calls.get(name, 0)
            self._calls[name] = call + 1
            for i, o in enumerate(outs):
                if isinstance(o, torch.Tensor):
                    rec = {"module": name, "call": call, "output": i, **tensor_stats(o)}
                    self._fh.write(json.dumps(rec) + "\n")
                    self._n += 1
        return fn

    def __enter__(self):
        self._fh = open(self.path, "w")
        for name, mod in self.model.named_modules():
            if name and (self.pattern is None or self.pattern.search(name)):
                self._handles.append(mod.register_forward_hook(self._hook(name)))
        return self

    def __exit__(self, *exc):
        for h in self._handles:
            h.remove()
        self._handles = []
        self._fh.close()
        return False


def load_dump(path: str) -> dict[tuple, dict]:
    out = {}
    with open(path) as f:
        for line in f:
            r = json.loads(line)
            out[(r["module"], r["call"], r["output"])] = r
    return out


def compare_dumps(path_a: str, path_b: str, rtol: float = 5e-2, atol: float = 1e-3) -> dict:
    """Rows whose l2 / absmax / mean differ beyond tolerance, in execution order of dump A; ``first`` is the first."""
    a, b = load_dump(path_a), load_dump(path_b)
    bad, missing = [], [k for k in a if k not in b]
    for k, ra in a.items():
        rb = b.get(k)
        if rb is None or ra.get("numel", 0) == 0:
            continue
        worst = 0.0
        for field in ("l2", "absmax", "mean"):
            x, y = ra[field], rb[field]
            err = abs(x - y) / (atol + rtol * max(abs(x), abs(y)))
            worst = max(worst, err)
        if worst > 1.0 or ra["nan"] != rb["nan"] or ra["inf"] != rb["inf"]:
            bad.append({"key": list(k), "a": {f: ra[f] for f in ("l2", "absmax", "mean", "nan", "inf")},
                        "b": {f: rb[f] for f in ("l2", "absmax", "mean", "nan", "inf")}, "excess": round(worst, 3)})
    return {"compared": len(a) - len(missing), "missing_in_b": len(missing), "mismatches": len(bad),
            "first": bad[0] if bad else None, "rows": bad[:50]}
