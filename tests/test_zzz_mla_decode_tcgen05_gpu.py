"""The tcgen05 absorbed-MLA decode kernel (csrc/mla_decode_tcgen05.cu) against the fp32 oracle.

The cases run in a child process: the file sorts last and the kernel is opt-in (``impl=2`` /
``B200_MLA_TCGEN05=1``), so whatever it does stays outside the process that runs the rest of the suite.  Cases: one and
two head tiles, fewer heads than a tile, lengths that end inside a tile / a page, several tokens per request, splits
that own no tile, page sizes 32 and 64, bf16 and fp16, and a score scale at which row maxima keep growing (the
accumulator rescale path).
"""
import json
import os
import subprocess
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

gpu = pytest.mark.gpu


def _mla_case(lens, qlens, H, bs, dtype, seed=0):
    g = torch.Generator().manual_seed(seed)
    B = len(lens)
    nblk = [(n + bs - 1) // bs for n in lens]
    total = sum(nblk) + 2
    perm = torch.randperm(total, generator=g)
    bt = torch.zeros(B, max(nblk), dtype=torch.int32)
    o = 0
    for b in range(B):
        bt[b, : nblk[b]] = perm[o:o + nblk[b]].to(torch.int32)
        o += nblk[b]
    cache = torch.randn(total * bs, 576, generator=g).to(dtype).view(total, bs, 576)
    q = (torch.randn(sum(qlens), H, 576, generator=g) * 0.3).to(dtype)
    qsl = torch.tensor([0] + list(torch.tensor(qlens).cumsum(0)), dtype=torch.int32)
    return q, cache, bt, torch.tensor(lens, dtype=torch.int32), qsl


CASES = [(H, splits, bs, scale, dt)
         for H in (128, 16, 200) for splits in (1, 3)
         for bs, scale, dt in ((64, 0.1, "bfloat16"), (32, 1.5, "bfloat16"), (64, 0.1, "float16"))]


def _child() -> None:
    from vllm_metax_b200 import _custom_ops as ops
    from vllm_metax_b200.ops import reference as ref

    ops.load_native()
    out = []
    for H, splits, bs, scale, dt in CASES:
        dtype = getattr(torch, dt)
        q, cache, bt, sl, qsl = _mla_case([70, 300, 17, 1000, 33], [1, 3, 1, 2, 1], H, bs, dtype, seed=5)
        lse = torch.empty(H, q.shape[0], device="cuda")
        got = ops.mla_decode(q.cuda(), cache.cuda(), bt.cuda(), sl.cuda(), scale, query_start_loc=qsl.cuda(),
                             lse_out=lse, num_splits=splits, impl=2)
        torch.cuda.synchronize()
        want, wlse = ref.mla_decode(q.float(), cache.float(), bt, sl, scale, query_start_loc=qsl)
        a, b = got.float().cpu().flatten(), want.flatten()
        cos = 1 - float(torch.dot(a, b) / (a.norm() * b.norm()))
        out.append({"case": [H, splits, bs, scale, dt], "finite": bool(torch.isfinite(a).all()), "cos_diff": cos,
                    "lse_max_diff": float((lse.cpu() - wlse).abs().max())})
    print("RESULT " + json.dumps({"cases": out, "status": ops.kernel_status()}))


@gpu
def test_mla_decode_tcgen05_against_oracle():
    r = subprocess.run([sys.executable, os.path.abspath(__file__), "--child"], capture_output=True, text=True,
                       timeout=600, cwd=ROOT)
    line = next((ln for ln in r.stdout.splitlines() if ln.startswith("RESULT ")), None)
    assert r.returncode == 0 and line is not None, (r.returncode, r.stdout[-2000:], r.stderr[-3000:])
    res = json.loads(line[len("RESULT "):])
    assert res["status"]["code"] == 0, res["status"]          # no bounded wait ran out, no index was out of range
    for c in res["cases"]:
        scale = c["case"][3]
        assert c["finite"], c
        assert c["cos_diff"] < (5e-4 if scale < 1 else 3e-3), c
        assert c["lse_max_diff"] < 5e-2 * max(1.0, scale * 10), c


if __name__ == "__main__" and "--child" in sys.argv:
    _child()
