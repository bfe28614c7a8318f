"""Fused compute + collective layers over NVLink peer memory.

``FusedRowParallelNorm`` is the tensor-parallel row-parallel linear (o_proj / down_proj) fused
with everything that follows it: GEMM -> reduce-scatter into the owning rank -> residual add
-> RMSNorm -> all-gather of the normalised rows.  Two implementations share one workspace:

``split`` (default)  the CTA-pair GEMM (prefill chunks) or the stream-K GEMM (decode batches) stores each output
                     row from its epilogue straight into the owning rank's receive slot over NVLink while the
                     tensor cores work on the next tile; ONE more kernel (``csrc/comm_ar_norm.cu``) then reduces,
                     adds the residual, normalises and all-gathers.  Two launches, no library collective.
``mono``             one kernel per rank for all of it (``csrc/comm_gemm_ar_norm.cu``, 128 x 256 single-CTA tiles).

Both replace GEMM + NCCL all-reduce + fused_add_rms_norm (the reference's path C1 -> K12, and its
quick-reduce / minimax_reduce_rms special cases).

The residual stream is kept sharded by token rows between calls: rank r owns rows
``[r * rows_per_rank, (r + 1) * rows_per_rank)`` of the step's ``T`` tokens.

On CPU tensors (Gloo ranks) the same contract is met with plain collectives, which is how the
host-side logic is tested without GPUs.
"""
from __future__ import annotations

from typing import Optional

import torch

from .. import _custom_ops as ops
from .. import envs
from ..ops import reference as ref
from .state import Group
from .symm_mem import SymmWorkspace


def rows_per_rank(T: int, tp: int) -> int:
    return (T + tp - 1) // tp


class FusedRowParallelNorm:
    """Workspace + launcher shared by every fused row-parallel layer of a model."""

    def __init__(self, group: Group, device: torch.device, max_tokens: int, hidden: int, dtype: torch.dtype):
        self.group, self.device, self.hidden, self.dtype = group, device, hidden, dtype
        self.tp, self.rank = group.world_size, group.rank_in_group
        self.max_tokens = max_tokens
        self.rows_cap = (rows_per_rank(max_tokens, self.tp) + 7) // 8 * 8
        self.rb_cap = (max_tokens + 127) // 128 + 1
        self.cuda = device.type == "cuda"
        self.kernel = (envs.B200_FUSED_TP_KERNEL or "split").lower()
        if not self.cuda:
            return
        esz = torch.empty((), dtype=dtype).element_size()
        n_recv = self.tp * self.rows_cap * hidden * esz
        n_out = max_tokens * hidden * esz
        n_cnt = 2 * self.rb_cap * 4
        n_flag = 64
        self.ws = SymmWorkspace(group, n_recv + n_out + n_cnt + 3 * n_flag + 12 * SymmWorkspace.ALIGN, device)
        r_recv = self.ws.region("recv", n_recv)
        r_cnt = self.ws.region("counters", n_cnt)
        r_flag = self.ws.region("flags", n_flag)
        r_out = self.ws.region("out", n_out)
        # flags of the split path: push epochs (written by the scatter GEMMs) and gather epochs
        r_f1, r_f2 = self.ws.region("push_flags", 64), self.ws.region("gather_flags", 64)
        self.ws.local(r_f1, torch.int32, (16,)).zero_()
        self.ws.local(r_f2, torch.int32, (16,)).zero_()
        self.out = self.ws.local(r_out, dtype, (max_tokens, hidden))
        self.ptrs = torch.tensor([self.ws.peer_ptrs(r_recv), self.ws.peer_ptrs(r_cnt), self.ws.peer_ptrs(r_flag),
                                  self.ws.peer_ptrs(r_out)], dtype=torch.int64)
        self.ptrs_scatter = torch.tensor([self.ws.peer_ptrs(r_recv), self.ws.peer_ptrs(r_f1)], dtype=torch.int64)
        self.ptrs_gather = torch.tensor([self.ws.peer_ptrs(r_recv), self.ws.peer_ptrs(r_f1), self.ws.peer_ptrs(r_f2),
                                         self.ws.peer_ptrs(r_out)], dtype=torch.int64)
        self.local_sync = torch.zeros(4, dtype=torch.int32, device=device)
        self.local_sync_split = torch.zeros(4, dtype=torch.int32, device=device)
        self.out_mc = 0
        self._ipc_out, self._ipc_ptrs_gather = self.out, self.ptrs_gather
        mm = int(envs.B200_USE_MULTIMEM)
        if (mm >= 2 or (mm == 1 and self.tp >= 4)) and self.tp > 1 and self.kernel != "mono":   # "mono" gathers through self.ptrs
            self._try_multicast_out(n_out, dtype, max_tokens, hidden, r_recv, r_f1, r_f2)
        self.wait_cycles = int(envs.B200_PEER_WAIT_ITERS) * 200  # iteration budget expressed in SM cycles
        self.nvls = None
        self.nvls_max_tokens = min(int(envs.B200_NVLS_AR_MAX_TOKENS), max_tokens)
        if mm >= 1 and self.tp > 1 and self.kernel != "mono" and self.nvls_max_tokens > 0:
            self._try_nvls(dtype, hidden)
        torch.cuda.synchronize(device)
        group.barrier()

    def _try_multicast_out(self, n_out, dtype, max_tokens, hidden, r_recv, r_f1, r_f2) -> None:
        """Puts the all-gathered output buffer into torch's symmetric memory, which binds the ranks' copies to ONE
        NVLink multicast address when the fabric supports it: the gather kernel then issues a single
        ``multimem.st`` per 16 bytes and the NVSwitch replicates it (1/tp of the bytes leave the GPU).  Any failure
        keeps the IPC buffer and the per-rank peer stores."""
        try:
            import torch.distributed._symmetric_memory as symm

            buf = symm.empty(n_out, dtype=torch.uint8, device=self.device)
            hdl = symm.rendezvous(buf, self.group.device_pg)
            mc = int(getattr(hdl, "multicast_ptr", 0) or 0)
            ptrs = [int(p) for p in hdl.buffer_ptrs]
            if mc == 0 or len(ptrs) != self.tp:
                return
            self._mc_buf, self._mc_hdl = buf, hdl
            self.out = buf.view(dtype).view(max_tokens, hidden)
            self.out_mc = mc
            self.ptrs_gather = torch.tensor([self.ws.peer_ptrs(r_recv), self.ws.peer_ptrs(r_f1),
                                             self.ws.peer_ptrs(r_f2), ptrs], dtype=torch.int64)
        except Exception:      # no multicast support in this torch build / driver / fabric
            self.out_mc = 0

    def _try_nvls(self, dtype, hidden) -> None:
        """Small steps (decode batches): a plain local GEMM into a multicast-mapped buffer, then ONE kernel that
        reduces through the switch (``multimem.ld_reduce``), adds the residual, normalises and writes every rank's
        output (``multimem.st``) - ``csrc/comm_nvls_ar_norm.cu``.  Needs torch symmetric memory with a multicast
        handle; without one the peer-store path serves every size."""
        try:
            import torch.distributed._symmetric_memory as symm

            esz = torch.empty((), dtype=dtype).element_size()
            n_buf = (self.nvls_max_tokens * hidden * esz + 1023) // 1024 * 1024
            buf = symm.empty(2 * n_buf + 1024, dtype=torch.uint8, device=self.device)
            buf.zero_()
            hdl = symm.rendezvous(buf, self.group.device_pg)
            mc = int(getattr(hdl, "multicast_ptr", 0) or 0)
            if mc == 0:
                return
            self.nvls = {
                "buf": buf, "hdl": hdl, "mc": mc,
                "partial": buf[:n_buf].view(dtype)[: self.nvls_max_tokens * hidden].view(self.nvls_max_tokens, hidden),
                "out": buf[n_buf: 2 * n_buf].view(dtype)[: self.nvls_max_tokens * hidden].view(self.nvls_max_tokens, hidden),
                "partial_mc": mc, "out_mc": mc + n_buf, "flag_mc": mc + 2 * n_buf,
                "flag_local": buf.data_ptr() + 2 * n_buf,
                "sync": torch.zeros(4, dtype=torch.int32, device=self.device),
            }
        except Exception:      # no multicast support in this torch build / driver / fabric
            self.nvls = None

    def disable_nvls(self) -> None:
        self.nvls = None

    def disable_multicast(self) -> None:
        """Back to the IPC output buffer and per-rank peer stores (start-up check failed with multicast on)."""
        self.out_mc = 0
        self.out, self.ptrs_gather = self._ipc_out, self._ipc_ptrs_gather

    def __call__(self, x: torch.Tensor, weight: torch.Tensor, residual_shard: torch.Tensor,
                 norm_weight: torch.Tensor, eps: float, add_residual: bool = True) -> torch.Tensor:
        """``x [T, K_local]``, ``weight [H, K_local]``; ``residual_shard [rows_per_rank(T), H]`` is updated in
        place (overwritten when ``add_residual`` is False).  Returns the normalised ``[T, H]`` (a view of the
        symmetric output buffer, valid until the next call)."""
        T = x.shape[0]
        rpr = rows_per_rank(T, self.tp)
        self.calls = getattr(self, "calls", 0) + 1
        if self.cuda:
            assert T <= self.max_tokens
            if self.kernel == "mono":
                ops._launches += 1
                torch.ops.b200.gemm_ar_norm(x, weight, residual_shard, norm_weight, eps, self.ptrs, self.tp, self.rank,
                                            rpr, self.rows_cap, self.rb_cap, self.local_sync, add_residual,
                                            self.wait_cycles)
                return self.out[:T]
            nv = self.nvls
            if nv is not None and T <= self.nvls_max_tokens:
                ops._launches += 2
                torch.ops.b200.gemm(nv["partial"][:T], x, weight, None, None, 0, 0)
                torch.ops.b200.nvls_ar_norm(residual_shard, norm_weight, eps, nv["partial_mc"], nv["out_mc"],
                                            nv["flag_mc"], nv["flag_local"], T, self.hidden, self.tp, self.rank, rpr,
                                            nv["sync"], add_residual, self.wait_cycles)
                return nv["out"][:T]
            ops._launches += 2
            torch.ops.b200.gemm_row_scatter(x, weight, self.ptrs_scatter, self.tp, self.rank, rpr, self.rows_cap,
                                            self.local_sync_split)
            torch.ops.b200.ar_norm_gather(residual_shard, norm_weight, eps, self.ptrs_gather, T, self.hidden, self.tp,
                                          self.rank, rpr, self.rows_cap, self.local_sync_split, add_residual,
                                          self.wait_cycles, self.out_mc)
            return self.out[:T]
        # CPU ranks: same contract through plain collectives
        part = ref.gemm(x, weight, out_dtype=torch.float32)
        part = part.to(x.dtype).float()              # partials travel in the activation dtype
        pad = rpr * self.tp - T
        if pad:
            part = torch.cat([part, part.new_zeros(pad, part.shape[1])])
        mine = self.group.reduce_scatter(part, 0)
        my_rows = max(0, min(rpr, T - self.rank * rpr))
        if add_residual:
            mine[:my_rows] += residual_shard[:my_rows].float()
        residual_shard[:my_rows] = mine[:my_rows].to(residual_shard.dtype)
        normed = ref.rms_norm(residual_shard[:rpr], norm_weight, eps)
        if normed.shape[0] < rpr:
            normed = torch.cat([normed, normed.new_zeros(rpr - normed.shape[0], normed.shape[1])])
        return self.group.all_gather(normed.contiguous(), 0)[:T]


    def self_test(self, tokens=(8, 300, 2100)) -> tuple[bool, str]:
        """Runs the fused path on random data at this world size and compares it with an fp32 statement of the same
        contract built from all-gathered inputs.  Returns (ok, reason); the verdict is the same on every rank.  A
        failed or timed-out kernel leaves the context usable (bounded waits set the status word, cleared here)."""
        if not self.cuda or self.tp == 1:
            return True, ""
        import torch.distributed as dist

        ok, why = True, ""
        K = 256
        gen = torch.Generator(device="cpu").manual_seed(4321)
        for T in tokens:
            T = min(T, self.max_tokens)
            # same generator on every rank: rank r uses slice r, and knows everybody's inputs
            xs = torch.randn(self.tp, T, K, generator=gen).to(self.device, self.dtype)
            wsl = (torch.randn(self.tp, self.hidden, K, generator=gen) * 0.05).to(self.device, self.dtype)
            res_full = torch.randn(self.tp * rows_per_rank(T, self.tp), self.hidden, generator=gen).to(self.device, self.dtype)
            nw = torch.randn(self.hidden, generator=gen).to(self.device, self.dtype)
            rpr = rows_per_rank(T, self.tp)
            res = res_full[self.rank * rpr:(self.rank + 1) * rpr].clone()
            got = self(xs[self.rank].contiguous(), wsl[self.rank].contiguous(), res, nw, 1e-5).float().clone()
            part = sum((xs[r].float() @ wsl[r].float().t()).to(self.dtype).float() for r in range(self.tp))
            new_res = (part + res_full[:T].float()).to(self.dtype)
            want = ref.rms_norm(new_res, nw, 1e-5).float()
            torch.cuda.synchronize(self.device)
            err = float((got - want).abs().max())
            lim = 0.06 * max(1.0, float(want.abs().max()))
            n_mine = max(0, min(rpr, T - self.rank * rpr))
            err_res = float((res[:n_mine].float() - new_res[self.rank * rpr:self.rank * rpr + n_mine].float()).abs().max()) if n_mine else 0.0
            if not (err <= lim and err_res <= lim):
                ok, why = False, f"numeric mismatch at T={T}: out {err:.3g}, residual {err_res:.3g} (limit {lim:.3g})"
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


_SHARED: dict = {}


def get_fused_row_parallel(group: Group, device: torch.device, max_tokens: int, hidden: int,
                           dtype: torch.dtype) -> FusedRowParallelNorm:
    key = (id(group), str(device), hidden, dtype)
    cur = _SHARED.get(key)
    if cur is None or cur.max_tokens < max_tokens:
        cur = FusedRowParallelNorm(group, device, max_tokens, hidden, dtype)
        _SHARED[key] = cur
    return cur


class AllGatherGemm:
    """``concat_r(x_r) @ W^T`` for row-sharded activations as ONE kernel per rank (``csrc/comm_ag_gemm.cu``):
    remote row blocks stream in over NVLink (once each) while the tensor cores already work on the local
    shard.  ``x_shard()`` is the symmetric input buffer the producing op writes into.

    On CPU tensors the same contract is met with an all-gather + matmul (host-side tests)."""

    def __init__(self, group: Group, device: torch.device, max_rows_per_rank: int, k: int, dtype: torch.dtype):
        self.group, self.device, self.k, self.dtype = group, device, k, dtype
        self.tp, self.rank = group.world_size, group.rank_in_group
        self.rows_cap = (max_rows_per_rank + 127) // 128 * 128
        self.cuda = device.type == "cuda"
        if not self.cuda:
            self._x = torch.zeros(self.rows_cap, k, dtype=dtype)
            return
        esz = torch.empty((), dtype=dtype).element_size()
        n_x = self.rows_cap * k * esz
        self.ws = SymmWorkspace(group, n_x + 3 * SymmWorkspace.ALIGN + 4096, device)
        r_x, r_ready, r_done = self.ws.region("ag_x", n_x), self.ws.region("ag_xready", 64), self.ws.region("ag_done", 64)
        self._x = self.ws.local(r_x, dtype, (self.rows_cap, k))
        self.ws.local(r_ready, torch.int32, (16,)).zero_()
        self.ws.local(r_done, torch.int32, (16,)).zero_()
        self.ptrs = torch.tensor([self.ws.peer_ptrs(r_x), self.ws.peer_ptrs(r_ready), self.ws.peer_ptrs(r_done)],
                                 dtype=torch.int64)
        self.gathered = torch.empty(self.tp * self.rows_cap, k, dtype=dtype, device=device)
        self.ready = torch.zeros(self.tp * self.rows_cap // 128 + 1, dtype=torch.int32, device=device)
        self.sync = torch.zeros(4, dtype=torch.int32, device=device)
        self.wait_cycles = int(envs.B200_PEER_WAIT_ITERS) * 200
        torch.cuda.synchronize(device)
        group.barrier()

    def x_shard(self, rows: int) -> torch.Tensor:
        """The first ``rows`` (multiple of 128) rows of this rank's symmetric input buffer."""
        assert rows % 128 == 0 and rows <= self.rows_cap
        return self._x[:rows]

    def __call__(self, rows: int, w: torch.Tensor, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
        """``rows`` = rows per rank (same on every rank, multiple of 128); returns ``[tp*rows, N]``."""
        if not self.cuda:
            x_all = self.group.all_gather(self._x[:rows], 0) if self.tp > 1 else self._x[:rows]
            y = x_all.float() @ w.float().t()
            if bias is not None:
                y = y + bias.float()
            return y.to(self.dtype)
        out = torch.empty(self.tp * rows, w.shape[0], dtype=self.dtype, device=self.device)
        # the shard buffer is [rows_cap, K] on every rank; with rows < rows_cap the kernel still addresses row
        # blocks relative to each shard's base, and the gathered buffer is indexed with `rows` per rank
        torch.ops.b200.ag_gemm(out, w, bias, self.ptrs, self.gathered, self.ready, self.sync, self.tp, self.rank,
                               rows, self.wait_cycles)
        return out

    def close(self) -> None:
        if self.cuda:
            self.ws.close()
