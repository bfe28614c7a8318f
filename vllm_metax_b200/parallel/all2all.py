"""Expert-parallel token exchange ("all2all managers").

Two implementations of one interface - ``dispatch`` tokens to the ranks owning their experts, run the
local experts, ``combine`` the outputs back with the top-k weights:

* ``NvlinkAll2AllManager``  hand-written kernels over peer-mapped symmetric memory (``csrc/comm_moe_a2a.cu``):
  one dispatch kernel (rows pushed with plain NVLink stores, optionally quantised to fp8 1x128 on the
  way) and a combine pair (send-back, then weighted top-k sum).  Receivers see
  ``recv_x [ep*cap, H]``, ``recv_ids [ep*cap]`` (local expert or -1) which feed ``moe_align`` unchanged.
* ``AgRsAll2AllManager``    collectives only (works on any backend, incl. Gloo on CPU): dispatch is an
  ``all_gatherv`` of the hidden states and ONE packed tensor ``[topk_weights | float(topk_ids) | scale]``
  - two collectives instead of three or four - combine a ``reduce_scatterv``.

``run_experts_a2a`` is the layer-level driver used by ``FusedMoE`` when tokens are sharded over the EP
group (sequence-parallel MoE).

Parity: vllm_metax/distributed/device_communicators/all2all.py:20-218 (MacaAgRsAll2AllManager packing
:64-142 / fused_unpack :96, MacaDeepEPLLAll2AllManager :163-218),
model_executor/layers/fused_moe/prepare_finalize/deepep_ll.py:24-145.
"""
from __future__ import annotations

from typing import Callable, Optional, Sequence

import torch

from .. import _custom_ops as ops
from .state import Group

WAIT_CYCLES = 4_000_000_000     # ~2 s of SM clock: a peer that never arrives becomes an error, not a hang


# ----------------------------------------------------------------------------- packed side-band tensor
def pack_routing(topk_weights: torch.Tensor, topk_ids: torch.Tensor, scale: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``[T, 2*topk (+n_scale)] f32 = [weights | float(ids) | scale]`` (ids < 2^24 are exact in f32)."""
    parts = [topk_weights.float(), topk_ids.float()]
    if scale is not None:
        parts.append(scale.float().reshape(topk_ids.shape[0], -1))
    return torch.cat(parts, dim=1).contiguous()


def unpack_routing(packed: torch.Tensor, topk: int, ids_dtype=torch.int32):
    """Inverse of ``pack_routing``: ``(weights f32, ids, scale or None)``."""
    w = packed[:, :topk].contiguous()
    ids = packed[:, topk:2 * topk].round().to(ids_dtype)
    scale = packed[:, 2 * topk:].contiguous() if packed.shape[1] > 2 * topk else None
    return w, ids, scale


class AgRsAll2AllManager:
    """All-gather / reduce-scatter token exchange."""

    def __init__(self, group: Group):
        self.group = group

    def dispatch(self, hidden: torch.Tensor, topk_weights: torch.Tensor, topk_ids: torch.Tensor,
                 sizes: Optional[Sequence[int]] = None, scale: Optional[torch.Tensor] = None):
        """Every rank ends up with the tokens of all ranks: ``(hidden_all, weights_all, ids_all, scale_all)``."""
        g = self.group
        if g.world_size == 1:
            return hidden, topk_weights, topk_ids, scale
        if sizes is None:
            sizes = [int(s) for s in g.all_gather_object(int(hidden.shape[0]))]
        self.sizes = list(sizes)
        topk = topk_ids.shape[1]
        packed = pack_routing(topk_weights, topk_ids, scale)
        h_all = g.all_gatherv(hidden.contiguous(), self.sizes)
        p_all = g.all_gatherv(packed, self.sizes)
        w, ids, sc = unpack_routing(p_all, topk, topk_ids.dtype)
        return h_all, w, ids, sc

    def combine(self, partial_out: torch.Tensor) -> torch.Tensor:
        """``partial_out [sum(sizes), H]`` (this rank's experts only) -> this rank's tokens, summed over ranks."""
        g = self.group
        if g.world_size == 1:
            return partial_out
        return g.reduce_scatterv(partial_out.contiguous(), self.sizes)


# ----------------------------------------------------------------------------- NVLink kernels
class NvlinkAll2AllManager:
    """Dispatch / combine by peer stores (``csrc/comm_moe_a2a.cu``).  A token is sent once per destination RANK
    with its top-k list rewritten for that rank, so the receiver runs the ordinary local fused-MoE path on
    ``(recv_x, recv_ids, recv_w)`` and returns one partial sum per received token."""

    REGIONS = ("recv_x", "recv_scale", "recv_ids", "recv_src", "recv_count", "disp_flag", "comb_x", "comb_flag",
               "recv_w")

    def __init__(self, group: Group, max_tokens_per_rank: int, hidden: int, topk: int, num_experts: int,
                 dtype: torch.dtype, device: torch.device, quant_fp8: bool = False, workspace=None):
        from .symm_mem import SymmWorkspace

        self.group, self.ep, self.rank = group, group.world_size, group.rank_in_group
        assert num_experts % self.ep == 0 and hidden % (128 if quant_fp8 else 8) == 0
        self.H, self.topk, self.E_local = hidden, topk, num_experts // self.ep
        self.dtype, self.device, self.quant = dtype, device, quant_fp8
        self.max_tokens = max_tokens_per_rank
        self.cap = max_tokens_per_rank               # a source sends a token to a destination at most once
        slots = self.ep * self.cap
        esz = 1 if quant_fp8 else 2
        sizes = {
            "recv_x": slots * hidden * esz, "recv_scale": slots * (hidden // 128) * 4 if quant_fp8 else 16,
            "recv_ids": slots * topk * 4, "recv_w": slots * topk * 4, "recv_src": slots * 4, "recv_count": 64,
            "disp_flag": 64, "comb_x": slots * hidden * 2, "comb_flag": 64,
        }
        total = sum((v + 1023) // 1024 * 1024 for v in sizes.values()) + 4096
        self.ws = workspace or SymmWorkspace(group, total, device)
        self.reg = {k: self.ws.region(f"a2a_{k}", sizes[k]) for k in self.REGIONS}
        self.ptrs = torch.tensor([self.ws.peer_ptrs(self.reg[k]) for k in self.REGIONS], dtype=torch.int64)
        self.recv_x = self.ws.local(self.reg["recv_x"], torch.uint8 if quant_fp8 else dtype, (slots, hidden))
        self.recv_scale = self.ws.local(self.reg["recv_scale"], torch.float32, (slots, hidden // 128)) if quant_fp8 else None
        self.recv_ids = self.ws.local(self.reg["recv_ids"], torch.int32, (slots, topk))
        self.recv_w = self.ws.local(self.reg["recv_w"], torch.float32, (slots, topk))
        self.recv_ids.fill_(-1)
        self.recv_w.zero_()
        for k in ("recv_count", "disp_flag", "comb_flag"):
            self.ws.local(self.reg[k], torch.int32, (16,)).zero_()
        self.local_sync = torch.zeros(32, dtype=torch.int32, device=device)
        torch.cuda.synchronize(device)
        group.barrier()

    def dispatch(self, x: torch.Tensor, topk_weights: torch.Tensor, topk_ids: torch.Tensor):
        """Push this rank's tokens to the ranks that own their experts; returns the receive views
        ``(recv_x [ep*cap, H], recv_scale, recv_ids [ep*cap, topk], recv_w [ep*cap, topk])`` (empty slots: ids -1)."""
        assert x.shape[0] <= self.max_tokens and x.shape[1] == self.H and x.dtype == self.dtype
        torch.ops.b200.moe_a2a_dispatch(x.contiguous(), topk_ids.int().contiguous(), topk_weights.float().contiguous(),
                                        self.ptrs, self.ep, self.rank, self.E_local, self.cap, self.quant,
                                        self.local_sync, WAIT_CYCLES)
        return self.recv_x, self.recv_scale, self.recv_ids, self.recv_w

    def combine(self, y_tok: torch.Tensor, topk_ids: torch.Tensor,
                shared_out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """``y_tok [ep*cap, H]`` = weighted partial sum of every receive slot -> this rank's tokens, summed over the
        ranks that computed a part of them (+ ``shared_out``)."""
        out = torch.empty(topk_ids.shape[0], self.H, dtype=self.dtype, device=self.device)
        torch.ops.b200.moe_a2a_combine(out, y_tok.contiguous(), topk_ids.int().contiguous(), shared_out, self.ptrs,
                                       self.ep, self.rank, self.E_local, self.cap, self.local_sync, WAIT_CYCLES)
        return out

    def close(self) -> None:
        self.ws.close()


def run_experts_a2a(mgr: NvlinkAll2AllManager, x: torch.Tensor, topk_weights: torch.Tensor, topk_ids: torch.Tensor,
                    experts_fn: Callable, shared_out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """dispatch -> align -> gather -> ``experts_fn(a, a_scale, block_expert, total)`` -> weighted sum per received
    token -> combine.

    ``experts_fn`` maps expert-sorted rows ``a [padded, H]`` (bf16, or fp8 with ``a_scale``) to outputs of the same
    row count (the two grouped GEMMs and the activation)."""
    recv_x, recv_scale, recv_ids, recv_w = mgr.dispatch(x, topk_weights, topk_ids)
    sorted_ids, block_expert, total, inv = ops.moe_align_block_size(recv_ids, 128, mgr.E_local, None, want_inverse=True)
    a = torch.empty(sorted_ids.numel(), recv_x.shape[1], dtype=recv_x.dtype, device=recv_x.device)
    torch.ops.b200.gather_rows(a, recv_x, sorted_ids, total, mgr.topk)
    a_scale = None
    if recv_scale is not None:
        a_scale = torch.empty(sorted_ids.numel(), recv_scale.shape[1], dtype=torch.float32, device=recv_x.device)
        torch.ops.b200.gather_rows(a_scale, recv_scale, sorted_ids, total, mgr.topk)
    y = experts_fn(a, a_scale, block_expert, total)
    y_tok = ops.moe_combine(y, recv_w, inv, recv_ids.shape[0], None)
    return mgr.combine(y_tok, topk_ids, shared_out)
