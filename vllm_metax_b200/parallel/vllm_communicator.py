"""Device communicator handed to vLLM's ``GroupCoordinator`` (``Platform.get_device_communicator_cls``).

Collectives go through the process group's NCCL backend; the expert-parallel token exchange is one of this
package's managers, selected by ``all2all_backend``: ``"nvlink"`` (peer-memory kernels) or
``"allgather_reducescatter"`` (two collectives with the packed side-band tensor).
Parity: vllm_metax/distributed/device_communicators/cuda_communicator.py:19-62 (MacaCommunicator swaps
the all2all manager)."""
from __future__ import annotations

from typing import Optional

import torch
import torch.distributed as dist

from .. import envs

try:
    from vllm.distributed.device_communicators.base_device_communicator import DeviceCommunicatorBase
except Exception:  # pragma: no cover
    class DeviceCommunicatorBase:  # type: ignore
        def __init__(self, cpu_group, device=None, device_group=None, unique_name: str = ""):
            self.cpu_group, self.device, self.device_group, self.unique_name = cpu_group, device, device_group, unique_name
            self.world_size = dist.get_world_size(cpu_group)
            self.rank_in_group = dist.get_rank(cpu_group)


class _GroupView:
    """The slice of ``parallel.state.Group`` the all2all managers use, over vLLM's process groups."""

    def __init__(self, comm: "B200Communicator"):
        self.c = comm
        self.world_size, self.rank_in_group = comm.world_size, comm.rank_in_group

    def all_gather_object(self, obj):
        out = [None] * self.world_size
        dist.all_gather_object(out, obj, group=self.c.cpu_group)
        return out

    def barrier(self):
        dist.barrier(group=self.c.cpu_group)

    def all_gatherv(self, x, sizes):
        return self.c.all_gatherv(x, 0, list(sizes))

    def reduce_scatterv(self, x, sizes):
        return self.c.reduce_scatterv(x, 0, list(sizes))


class B200Communicator(DeviceCommunicatorBase):
    def __init__(self, cpu_group, device: Optional[torch.device] = None, device_group=None, unique_name: str = ""):
        super().__init__(cpu_group, device, device_group, unique_name)
        self.all2all_manager = None
        self.all2all_backend = "allgather_reducescatter" if not envs.B200_OPTIMIZED_DP_ALL2ALL else "nvlink"

    # ---- collectives (NCCL through torch.distributed) ----
    def all_reduce(self, x: torch.Tensor) -> torch.Tensor:
        out = x.clone()
        dist.all_reduce(out, group=self.device_group)
        return out

    def all_gather(self, x: torch.Tensor, dim: int = -1) -> torch.Tensor:
        if dim < 0:
            dim += x.dim()
        out = torch.empty((self.world_size,) + tuple(x.shape), dtype=x.dtype, device=x.device)
        dist.all_gather_into_tensor(out, x.contiguous(), group=self.device_group)
        return out.movedim(0, dim).reshape(*x.shape[:dim], self.world_size * x.shape[dim], *x.shape[dim + 1:])

    def all_gatherv(self, x, dim: int = 0, sizes: Optional[list[int]] = None):
        assert dim == 0
        if sizes is None:
            return self.all_gather(x, 0)
        outs = [torch.empty((s,) + tuple(x.shape[1:]), dtype=x.dtype, device=x.device) for s in sizes]
        dist.all_gather(outs, x.contiguous(), group=self.device_group)
        return torch.cat(outs, 0)

    def reduce_scatter(self, x: torch.Tensor, dim: int = -1) -> torch.Tensor:
        if dim < 0:
            dim += x.dim()
        xt = x.movedim(dim, 0).contiguous()
        out = torch.empty((xt.shape[0] // self.world_size,) + tuple(xt.shape[1:]), dtype=x.dtype, device=x.device)
        dist.reduce_scatter_tensor(out, xt, group=self.device_group)
        return out.movedim(0, dim)

    def reduce_scatterv(self, x: torch.Tensor, dim: int = 0, sizes: Optional[list[int]] = None) -> torch.Tensor:
        assert dim == 0
        if sizes is None:
            return self.reduce_scatter(x, 0)
        chunks = list(torch.split(x.contiguous(), sizes, 0))
        out = torch.empty_like(chunks[self.rank_in_group])
        dist.reduce_scatter(out, chunks, group=self.device_group)
        return out

    def send(self, x: torch.Tensor, dst: Optional[int] = None) -> None:
        dst = (self.rank_in_group + 1) % self.world_size if dst is None else dst
        dist.send(x, dist.get_global_rank(self.device_group, dst), group=self.device_group)

    def recv(self, size, dtype, src: Optional[int] = None) -> torch.Tensor:
        src = (self.rank_in_group - 1) % self.world_size if src is None else src
        x = torch.empty(size, dtype=dtype, device=self.device)
        dist.recv(x, dist.get_global_rank(self.device_group, src), group=self.device_group)
        return x

    def broadcast(self, x: torch.Tensor, src: int = 0) -> torch.Tensor:
        dist.broadcast(x, dist.get_global_rank(self.device_group, src), group=self.device_group)
        return x

    # ---- expert-parallel exchange ----
    def prepare_communication_buffer_for_model(self, model: torch.nn.Module) -> None:
        from .all2all import AgRsAll2AllManager

        if self.all2all_manager is None:
            self.all2all_manager = AgRsAll2AllManager(_GroupView(self))

    def dispatch(self, hidden_states, topk_weights, topk_ids, is_sequence_parallel: bool = False, extra_tensors=None):
        if self.all2all_manager is None:
            self.prepare_communication_buffer_for_model(None)
        h, w, ids, _ = self.all2all_manager.dispatch(hidden_states, topk_weights, topk_ids)
        return h, w, ids

    def combine(self, hidden_states, is_sequence_parallel: bool = False):
        return self.all2all_manager.combine(hidden_states)

    def destroy(self) -> None:
        self.all2all_manager = None
