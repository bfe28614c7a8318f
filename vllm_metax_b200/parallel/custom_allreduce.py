"""Stand-alone NVLink collectives for reductions that no GEMM precedes (``csrc/comm_allreduce.cu``).

``CustomAllReduce``   one-shot / two-shot all-reduce by peer stores into symmetric buffers; bit-identical results on
                      every rank (sources are summed in rank order).  ``Group.all_reduce`` routes CUDA tensors up to
                      ``max_bytes`` through it once ``attach()`` has been called; larger ones stay on NCCL.
``CrossRankRMSNorm``  RMSNorm over a hidden dimension that is split across ranks: only the per-token sums of squares
                      cross NVLink (4 bytes per token per peer, the value is its own arrival flag).

CPU tensors (Gloo ranks) take plain collectives with the same results, which is how the host logic is tested.

Parity: the reference's quick all-reduce (csrc/quickreduce/quick_reduce.h:69-195, two-shot with flags over IPC
buffers) and its Lamport reduce-RMS op (vllm_metax/registry/custom_ops/layers/minimax_rms_norm/
lamport_workspace.py:141-232, csrc/minimax_reduce_rms_kernel.cu:237-599).
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from .. import _custom_ops as ops
from .. import envs
from .state import Group
from .symm_mem import SymmWorkspace

_DTYPES = (torch.bfloat16, torch.float16, torch.float32)
MAX_CTAS = 160


class CustomAllReduce:
    def __init__(self, group: Group, device: torch.device, max_bytes: int = 8 << 20):
        self.group, self.device = group, device
        self.tp, self.rank = group.world_size, group.rank_in_group
        self.max_bytes = (max_bytes + 1023) // 1024 * 1024
        self.cuda = device.type == "cuda" and self.tp > 1
        if not self.cuda:
            return
        n_recv = 2 * self.tp * self.max_bytes
        n_gather = 2 * self.max_bytes
        n_flag = self.tp * MAX_CTAS * 4
        self.ws = SymmWorkspace(group, n_recv + n_gather + 2 * n_flag + 8 * SymmWorkspace.ALIGN, device)
        regions = [self.ws.region("ar_recv", n_recv), self.ws.region("ar_gather", n_gather),
                   self.ws.region("ar_flag1", n_flag), self.ws.region("ar_flag2", n_flag)]
        self.ws.local(regions[2], torch.int32, (self.tp * MAX_CTAS,)).zero_()
        self.ws.local(regions[3], torch.int32, (self.tp * MAX_CTAS,)).zero_()
        self.ptrs = torch.tensor([self.ws.peer_ptrs(r) for r in regions], dtype=torch.int64)
        self.local_sync = torch.zeros(4, dtype=torch.int32, device=device)
        self.wait_cycles = int(envs.B200_PEER_WAIT_ITERS) * 200
        torch.cuda.synchronize(device)
        group.barrier()

    def supports(self, x: torch.Tensor) -> bool:
        n = x.numel() * x.element_size()
        return (self.cuda and x.is_cuda and x.dtype in _DTYPES and x.is_contiguous() and 0 < n <= self.max_bytes
                and n % 16 == 0)

    def all_reduce(self, x: torch.Tensor, out: Optional[torch.Tensor] = None, mode: int = 0) -> torch.Tensor:
        """Sum over the group.  ``mode``: 0 picks by size, 1 forces one-shot, 2 two-shot.  In place when ``out`` is
        None (the kernel reads its input before any rank can overwrite it: inputs are pushed first)."""
        if self.tp == 1:
            return x
        if not x.is_cuda:
            return self.group.all_reduce(x)
        assert self.supports(x), "tensor not eligible for the NVLink all-reduce"
        out = x if out is None else out
        ops._launches += 1
        torch.ops.b200.custom_allreduce(out, x, self.ptrs, self.tp, self.rank, self.max_bytes, MAX_CTAS,
                                        self.local_sync, mode, self.wait_cycles)
        return out

    def self_test(self) -> tuple[bool, str]:
        """Both modes on a small and a medium message against the fp32 sum of the all-gathered inputs (the library
        all-reduce rounds between its steps, so its 16-bit result is not an exact oracle beyond two ranks).  The
        tolerance is one 16-bit rounding of the largest possible sum.  Returns (ok, reason); every rank gets the
        same verdict (the comparison result is itself reduced).  A failed or timed-out kernel leaves the context
        usable: the waits are bounded and only set the status word, which is cleared here."""
        if not self.cuda:
            return True, ""
        import torch.distributed as dist

        ok, why = True, ""
        gen = torch.Generator(device="cpu").manual_seed(1234)
        for n in (4096, min(self.max_bytes // 2, 1 << 20)):
            allx = torch.randn(self.tp, n, generator=gen).to(self.device, torch.bfloat16)   # same on every rank
            x = allx[self.rank].contiguous()
            want = allx.float().sum(0)
            lim = float(want.abs().max()) * 2.0 ** -7 + 1e-3
            for mode in (1, 2):
                got = torch.empty_like(x)
                self.all_reduce(x, out=got, mode=mode)
                err = float((got.float() - want).abs().max())
                if not err <= lim:
                    ok, why = False, f"numeric mismatch, {n} elements mode {mode}: {err:.3g} > {lim:.3g}"
        torch.cuda.synchronize(self.device)
        try:
            ops.check_kernel_status(self.device.index or 0)
        except RuntimeError as e:
            ok, why = False, f"kernel status: {e}"
        flag = torch.tensor([1 if ok else 0], device=self.device, dtype=torch.int32)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN, group=self.group.device_pg)
        all_ok = bool(flag.item())
        if not all_ok and ok:
            why = "another rank failed the check"
        return all_ok, why

    def attach(self) -> None:
        """Make ``group.all_reduce`` use this object for eligible CUDA tensors."""
        self.group.custom_allreduce = self

    def close(self) -> None:
        if getattr(self.group, "custom_allreduce", None) is self:
            self.group.custom_allreduce = None
        if self.cuda:
            self.ws.close()


class CrossRankRMSNorm:
    """``y = x * rsqrt(mean over the FULL hidden dimension of x^2 + eps) * w`` where each rank holds a slice of the
    hidden dimension (``x [T, H_local]``).  ``__call__`` normalises one tensor or a (q, k) pair in one launch."""

    def __init__(self, group: Group, device: torch.device, max_tokens: int):
        self.group, self.device = group, device
        self.tp, self.rank = group.world_size, group.rank_in_group
        self.t_cap = max_tokens
        self.cuda = device.type == "cuda" and self.tp > 1
        if not self.cuda:
            return
        n = 3 * 2 * self.tp * self.t_cap * 4
        self.ws = SymmWorkspace(group, n + 2 * SymmWorkspace.ALIGN, device)
        r = self.ws.region("rms_slots", n)
        # -0.0 everywhere: "not written yet"
        self.ws.local(r, torch.int32, (n // 4,)).fill_(-(1 << 31))
        self.ptrs = torch.tensor(self.ws.peer_ptrs(r), dtype=torch.int64)
        self.local_sync = torch.zeros(8, dtype=torch.int32, device=device)
        self.wait_cycles = int(envs.B200_PEER_WAIT_ITERS) * 200
        torch.cuda.synchronize(device)
        group.barrier()

    def _one_cpu(self, x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
        ss = x.float().pow(2).sum(-1, keepdim=True)
        if self.tp > 1:
            ss = self.group.all_reduce(ss)
        inv = torch.rsqrt(ss / (x.shape[-1] * self.tp) + eps)
        return (x.float() * inv * w.float()).to(x.dtype)

    def __call__(self, x: torch.Tensor, w: torch.Tensor, eps: float, x2: Optional[torch.Tensor] = None,
                 w2: Optional[torch.Tensor] = None) -> Tuple[torch.Tensor, Optional[torch.Tensor]]:
        if not (self.cuda and x.is_cuda):
            return self._one_cpu(x, w, eps), (self._one_cpu(x2, w2, eps) if x2 is not None else None)
        assert x.shape[0] <= self.t_cap
        x = x if x.stride(0) == x.shape[1] else x.contiguous()
        out = torch.empty_like(x)
        out2 = None
        if x2 is not None:
            x2 = x2 if x2.stride(0) == x2.shape[1] else x2.contiguous()
            out2 = torch.empty_like(x2)
        ops._launches += 1
        torch.ops.b200.reduce_rms(out, x, w, out2, x2, w2, eps, self.ptrs, self.tp, self.rank, self.t_cap,
                                  self.local_sync, self.wait_cycles)
        return out, out2

    def close(self) -> None:
        if self.cuda:
            self.ws.close()
