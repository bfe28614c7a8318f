"""Process-group bookkeeping: one process per GPU, NCCL for device collectives, Gloo for control.

World layout (rank = pp * tp_size + tp): TP ranks are adjacent so that on one
NVSwitch box a TP group is any aligned run of GPUs.  EP reuses the TP*DP ranks
(experts are sharded over the same processes that shard attention heads), DCP
subdivides TP.  With world_size == 1 every group is a trivial ``Group`` whose
collectives are identities, so model code never branches on "is distributed".

Parity: the reference inherits vllm.distributed.parallel_state (_TP/_PP/_DP/_EP/_DCP)
and plugs ``MacaCommunicator`` into GroupCoordinator
(vllm_metax/distributed/device_communicators/cuda_communicator.py:19-62).
"""
from __future__ import annotations

import os
from dataclasses import dataclass
from typing import Optional, Sequence

import torch
import torch.distributed as dist


class Group:
    """A communicator over ``ranks`` (global ranks); wraps a torch ProcessGroup."""

    def __init__(self, ranks: Sequence[int], rank: int, device_pg=None, cpu_pg=None, name: str = ""):
        self.ranks = list(ranks)
        self.world_size = len(self.ranks)
        self.rank_in_group = self.ranks.index(rank) if rank in self.ranks else -1
        self.device_pg = device_pg
        self.cpu_pg = cpu_pg
        self.name = name
        self.custom_allreduce = None     # parallel.custom_allreduce.CustomAllReduce once attached

    # ---- collectives -----------------------------------------------------
    def all_reduce(self, x: torch.Tensor) -> torch.Tensor:
        if self.world_size == 1:
            return x
        car = self.custom_allreduce
        if car is not None and car.supports(x):
            return car.all_reduce(x)
        dist.all_reduce(x, group=self._pg(x))
        return x

    def all_gather(self, x: torch.Tensor, dim: int = -1) -> torch.Tensor:
        if self.world_size == 1:
            return x
        if dim < 0:
            dim += x.dim()
        xc = x.contiguous() if x.dim() else x.reshape(1)
        flat = torch.empty((self.world_size * xc.shape[0],) + tuple(xc.shape[1:]), dtype=x.dtype, device=x.device)
        dist.all_gather_into_tensor(flat, xc, group=self._pg(x))
        out = flat.view((self.world_size,) + tuple(x.shape)).movedim(0, dim)
        shp = list(x.shape)
        shp[dim] *= self.world_size
        return out.reshape(shp)

    def all_gatherv(self, x: torch.Tensor, sizes: Sequence[int]) -> torch.Tensor:
        """Concatenate dim-0 shards of differing length (``sizes[r]`` rows from rank r)."""
        if self.world_size == 1:
            return x
        mx = max(sizes)
        pad = torch.zeros((mx,) + tuple(x.shape[1:]), dtype=x.dtype, device=x.device)
        pad[: x.shape[0]] = x
        flat = torch.empty((self.world_size * mx,) + tuple(x.shape[1:]), dtype=x.dtype, device=x.device)
        dist.all_gather_into_tensor(flat, pad, group=self._pg(x))
        out = flat.view((self.world_size, mx) + tuple(x.shape[1:]))
        return torch.cat([out[r, : sizes[r]] for r in range(self.world_size)], dim=0)

    def reduce_scatter(self, x: torch.Tensor, dim: int = 0) -> torch.Tensor:
        if self.world_size == 1:
            return x
        xm = x.movedim(dim, 0).contiguous()
        n = xm.shape[0] // self.world_size
        if not x.is_cuda:  # Gloo has no reduce-scatter
            dist.all_reduce(xm, group=self.cpu_pg)
            return xm[self.rank_in_group * n:(self.rank_in_group + 1) * n].movedim(0, dim)
        out = torch.empty((n,) + tuple(xm.shape[1:]), dtype=x.dtype, device=x.device)
        dist.reduce_scatter_tensor(out, xm, group=self._pg(x))
        return out.movedim(0, dim)

    def reduce_scatterv(self, x: torch.Tensor, sizes: Sequence[int]) -> torch.Tensor:
        if self.world_size == 1:
            return x
        mx = max(sizes)
        buf = torch.zeros((self.world_size, mx) + tuple(x.shape[1:]), dtype=x.dtype, device=x.device)
        off = 0
        for r, s in enumerate(sizes):
            buf[r, :s] = x[off: off + s]
            off += s
        if not x.is_cuda:  # Gloo has no reduce-scatter
            dist.all_reduce(buf, group=self.cpu_pg)
            return buf[self.rank_in_group, : sizes[self.rank_in_group]].contiguous()
        out = torch.empty((mx,) + tuple(x.shape[1:]), dtype=x.dtype, device=x.device)
        dist.reduce_scatter_tensor(out, buf.view((self.world_size * mx,) + tuple(x.shape[1:])), group=self._pg(x))
        return out[: sizes[self.rank_in_group]]

    def broadcast(self, x: torch.Tensor, src: int = 0) -> torch.Tensor:
        if self.world_size > 1:
            dist.broadcast(x, src=self.ranks[src], group=self._pg(x))
        return x

    def broadcast_async(self, x: torch.Tensor, src: int = 0):
        """Start a broadcast; the returned work's ``wait()`` orders the current stream (NCCL) or the host (Gloo) after it."""
        return dist.broadcast(x, src=self.ranks[src], group=self._pg(x), async_op=True)

    def isend(self, x: torch.Tensor, dst: int):
        return dist.isend(x, dst=self.ranks[dst], group=self._pg(x))

    def irecv(self, x: torch.Tensor, src: int):
        return dist.irecv(x, src=self.ranks[src], group=self._pg(x))

    def send(self, x: torch.Tensor, dst: int) -> None:
        dist.send(x, dst=self.ranks[dst], group=self._pg(x))

    def recv(self, x: torch.Tensor, src: int) -> torch.Tensor:
        dist.recv(x, src=self.ranks[src], group=self._pg(x))
        return x

    def all_gather_object(self, obj):
        if self.world_size == 1:
            return [obj]
        out = [None] * self.world_size
        dist.all_gather_object(out, obj, group=self.cpu_pg)
        return out

    def barrier(self) -> None:
        if self.world_size > 1:
            dist.barrier(group=self.cpu_pg)

    def _pg(self, x: torch.Tensor):
        return self.device_pg if x.is_cuda else self.cpu_pg

    @property
    def is_first_rank(self) -> bool:
        return self.rank_in_group == 0

    @property
    def is_last_rank(self) -> bool:
        return self.rank_in_group == self.world_size - 1


@dataclass
class _State:
    rank: int = 0
    world_size: int = 1
    local_rank: int = 0
    tp: Optional[Group] = None
    pp: Optional[Group] = None
    dp: Optional[Group] = None
    ep: Optional[Group] = None
    dcp: Optional[Group] = None
    pcp: Optional[Group] = None
    world: Optional[Group] = None
    initialized: bool = False


_S = _State()


def _trivial(name: str) -> Group:
    return Group([0], 0, name=name)


def _pg_timeout():
    """Collective timeout from B200_PG_TIMEOUT_S (seconds): a short value turns a peer that never joins a
    collective into an error on the waiting ranks instead of a long stall."""
    import datetime

    v = os.environ.get("B200_PG_TIMEOUT_S")
    return datetime.timedelta(seconds=float(v)) if v else None


def init_distributed(tensor_parallel_size: int = 1, pipeline_parallel_size: int = 1, data_parallel_size: int = 1,
                     decode_context_parallel_size: int = 1, backend: Optional[str] = None,
                     device: Optional[str] = None, prefill_context_parallel_size: int = 1) -> None:
    """Create the process groups.  Reads RANK / WORLD_SIZE / LOCAL_RANK / MASTER_* from the environment.
    ``prefill_context_parallel_size`` adds an outer dimension of full (tensor-parallel) model copies that split the
    tokens of every prefill chunk between them; it is not combined with pipeline or data parallelism."""
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", str(rank)))
    _S.rank, _S.world_size, _S.local_rank = rank, world, local_rank
    if world == 1:
        _S.tp = _trivial("tp"); _S.pp = _trivial("pp"); _S.dp = _trivial("dp"); _S.ep = _trivial("ep")
        _S.dcp = _trivial("dcp"); _S.pcp = _trivial("pcp"); _S.world = _trivial("world")
        _S.initialized = True
        return
    use_cuda = (device or "cuda") == "cuda" and torch.cuda.is_available()
    if use_cuda:
        torch.cuda.set_device(local_rank)
    if not dist.is_initialized():
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29511")
        be = backend or ("cpu:gloo,cuda:nccl" if use_cuda else "gloo")
        kw = {}
        if use_cuda:
            kw["device_id"] = torch.device("cuda", local_rank)
        if _pg_timeout() is not None:
            kw["timeout"] = _pg_timeout()
        dist.init_process_group(backend=be, rank=rank, world_size=world, **kw)
    tp, pp, dp = tensor_parallel_size, pipeline_parallel_size, data_parallel_size
    pcp = prefill_context_parallel_size
    assert tp * pp * dp * pcp == world, f"tp*pp*dp*pcp = {tp * pp * dp * pcp} != world size {world}"
    assert pcp == 1 or (pp == 1 and dp == 1), "prefill context parallelism is combined with tensor parallelism only"

    def make(groups: list[list[int]], name: str) -> Group:
        mine = None
        for ranks in groups:
            if len(ranks) == 1:
                g = Group(ranks, rank, name=name) if rank in ranks else None
            else:
                tkw = {"timeout": _pg_timeout()} if _pg_timeout() is not None else {}
                dpg = dist.new_group(ranks, backend="nccl", **tkw) if use_cuda else None
                cpg = dist.new_group(ranks, backend="gloo", **tkw)
                g = Group(ranks, rank, dpg if use_cuda else cpg, cpg, name) if rank in ranks else None
            if g is not None:
                mine = g
        return mine

    # rank = (dp_idx * pp + pp_idx) * tp + tp_idx; with prefill context parallelism rank = pcp_idx * tp + tp_idx
    if pcp > 1:
        _S.pcp = make([[c * tp + t for c in range(pcp)] for t in range(tp)], "pcp")
        dp = pcp            # the tensor-parallel groups below are cut out of the world the same way
    else:
        _S.pcp = Group([rank], rank, name="pcp")
    tp_groups = [[(d * pp + p) * tp + t for t in range(tp)] for d in range(dp) for p in range(pp)]
    pp_groups = [[(d * pp + p) * tp + t for p in range(pp)] for d in range(dp) for t in range(tp)]
    dp_groups = [[(d * pp + p) * tp + t for d in range(dp)] for p in range(pp) for t in range(tp)]
    ep_groups = [[(d * pp + p) * tp + t for d in range(dp) for t in range(tp)] for p in range(pp)]
    _S.tp = make(tp_groups, "tp")
    _S.pp = make(pp_groups, "pp")
    if pcp > 1:             # the copies are not data-parallel replicas: they work on the same requests
        _S.dp = Group([rank], rank, name="dp")
        _S.ep = _S.tp
    else:
        _S.dp = make(dp_groups, "dp")
        _S.ep = make(ep_groups, "ep")
    dcp = decode_context_parallel_size
    if dcp > 1:
        assert tp % dcp == 0
        dcp_groups = [g[i: i + dcp] for g in tp_groups for i in range(0, tp, dcp)]
        _S.dcp = make(dcp_groups, "dcp")
    else:
        _S.dcp = Group([rank], rank, name="dcp")
    _S.world = Group(list(range(world)), rank, dist.group.WORLD, dist.new_group(list(range(world)), backend="gloo"), "world")
    _S.initialized = True


def ensure_initialized() -> None:
    if not _S.initialized:
        init_distributed()


def destroy() -> None:
    if dist.is_initialized():
        dist.destroy_process_group()
    global _S
    _S.__init__()


_MAX_TOKENS_PER_STEP = 8192


def set_max_tokens_per_step(n: int) -> None:
    """The scheduler's token budget of one step: collectively created buffers whose size must not depend on a
    replica's current batch (the expert-parallel receive slots) are sized from it."""
    global _MAX_TOKENS_PER_STEP
    _MAX_TOKENS_PER_STEP = int(n)


def max_tokens_per_step() -> int:
    return _MAX_TOKENS_PER_STEP


_NUM_REDUNDANT_EXPERTS = 0
_EPLB_ENABLED = False


def set_eplb(enabled: bool, num_redundant_experts: int = 0) -> None:
    """Expert-parallel load balancing for the MoE layers built from now on: ``num_redundant_experts`` extra expert
    slots over the EP group (parallel/eplb.py).  Set by the engine before the model is constructed."""
    global _NUM_REDUNDANT_EXPERTS, _EPLB_ENABLED
    _EPLB_ENABLED = bool(enabled)
    _NUM_REDUNDANT_EXPERTS = int(num_redundant_experts) if enabled else 0


_MOE_SEQUENCE_PARALLEL = False
_ALL2ALL_BACKEND = "fused_nvlink"


def set_moe_parallel(sequence_parallel: bool, all2all_backend: str = "fused_nvlink") -> None:
    """How the MoE layers built from now on exchange tokens inside one replica (``ParallelConfig``)."""
    global _MOE_SEQUENCE_PARALLEL, _ALL2ALL_BACKEND
    if all2all_backend not in ("fused_nvlink", "allgather_reducescatter"):
        raise ValueError(f"unknown all2all_backend {all2all_backend!r}")
    _MOE_SEQUENCE_PARALLEL, _ALL2ALL_BACKEND = bool(sequence_parallel), all2all_backend


def moe_sequence_parallel() -> bool:
    return _MOE_SEQUENCE_PARALLEL


def all2all_backend() -> str:
    return _ALL2ALL_BACKEND


def eplb_enabled() -> bool:
    return _EPLB_ENABLED


def num_redundant_experts() -> int:
    return _NUM_REDUNDANT_EXPERTS


def get_tp_group() -> Group:
    ensure_initialized(); return _S.tp


def get_pp_group() -> Group:
    ensure_initialized(); return _S.pp


def get_dp_group() -> Group:
    ensure_initialized(); return _S.dp


def get_ep_group() -> Group:
    ensure_initialized(); return _S.ep


def get_dcp_group() -> Group:
    ensure_initialized(); return _S.dcp


def get_pcp_group() -> Group:
    ensure_initialized(); return _S.pcp


def get_world_group() -> Group:
    ensure_initialized(); return _S.world


def tp_rank() -> int:
    return get_tp_group().rank_in_group


def tp_size() -> int:
    return get_tp_group().world_size


def global_rank() -> int:
    return _S.rank


def local_rank() -> int:
    return _S.local_rank


def tensor_model_parallel_all_reduce(x):
    return get_tp_group().all_reduce(x)


def tensor_model_parallel_all_gather(x, dim=-1):
    return get_tp_group().all_gather(x, dim)


def tensor_model_parallel_reduce_scatter(x, dim=0):
    return get_tp_group().reduce_scatter(x, dim)
