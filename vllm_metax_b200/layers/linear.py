"""Tensor-parallel linear layers.

``ColumnParallelLinear`` shards the output features, ``RowParallelLinear`` the
input features (its partial results are summed over the TP group),
``MergedColumnParallelLinear`` / ``QKVParallelLinear`` fuse several column-parallel
projections into one GEMM.  The matmul itself is delegated to a *quant method*
(``UnquantizedLinearMethod`` = the tcgen05 bf16 GEMM; fp8 block-scaled, int8 W8A8,
AWQ/GPTQ W4A16 live in ``quantization/``), selected per layer by the model's
quantisation config - the same split the reference inherits from upstream
(vllm ``LinearBase``/``LinearMethodBase``; quant dispatch at
vllm_metax/registry/quant_config/fp8.py:47-94).

``RowParallelLinear.forward_fused`` is the entry to the fused
GEMM -> NVLink all-reduce -> residual add -> RMSNorm kernel.
"""
from __future__ import annotations

from typing import Optional, Sequence

import torch
import torch.nn as nn

from .. import _custom_ops as ops
from ..parallel import state as ps


class LinearMethodBase:
    """Creates a layer's weights and applies them."""

    def create_weights(self, layer: "LinearBase", in_features: int, out_features: int, dtype: torch.dtype) -> None:
        raise NotImplementedError

    def apply(self, layer: "LinearBase", x: torch.Tensor, bias: Optional[torch.Tensor] = None,
              residual: Optional[torch.Tensor] = None) -> torch.Tensor:
        raise NotImplementedError

    def process_weights_after_loading(self, layer: "LinearBase") -> None:
        pass


class UnquantizedLinearMethod(LinearMethodBase):
    def create_weights(self, layer, in_features, out_features, dtype):
        layer.weight = nn.Parameter(torch.empty(out_features, in_features, dtype=dtype), requires_grad=False)

    def apply(self, layer, x, bias=None, residual=None):
        return ops.gemm(x, layer.weight, bias, residual)


class LinearBase(nn.Module):
    def __init__(self, in_features: int, out_features: int, bias: bool, dtype: torch.dtype,
                 quant_method: Optional[LinearMethodBase] = None, prefix: str = ""):
        super().__init__()
        self.in_features = in_features
        self.out_features = out_features
        self.prefix = prefix
        self.quant_method = quant_method or UnquantizedLinearMethod()
        self.dtype = dtype

    def _make(self, in_local: int, out_local: int, bias: bool) -> None:
        self.in_local, self.out_local = in_local, out_local
        self.quant_method.create_weights(self, in_local, out_local, self.dtype)
        self.bias = nn.Parameter(torch.zeros(out_local, dtype=self.dtype), requires_grad=False) if bias else None

    def _x2d(self, x: torch.Tensor):
        return x.reshape(-1, x.shape[-1]), x.shape[:-1]


def _expand_scalar(param, loaded: torch.Tensor, rows: int) -> torch.Tensor:
    """A per-tensor scale stored for a per-channel parameter: give every one of ``rows`` channels the value."""
    if getattr(param, "expand_scalar", False) and loaded.numel() == 1:
        return loaded.reshape(1, 1).expand(rows, 1)
    return loaded.reshape(-1, 1) if getattr(param, "expand_scalar", False) and loaded.dim() == 1 else loaded


class ReplicatedLinear(LinearBase):
    def __init__(self, in_features, out_features, bias=False, dtype=torch.bfloat16, quant_method=None, prefix=""):
        super().__init__(in_features, out_features, bias, dtype, quant_method, prefix)
        self._make(in_features, out_features, bias)

    def weight_loader(self, param: torch.Tensor, loaded: torch.Tensor, shard_id=None) -> None:
        loaded = _expand_scalar(param, loaded, self.out_features)
        param.data.copy_(loaded.reshape(param.shape))

    def forward(self, x):
        x2, lead = self._x2d(x)
        return self.quant_method.apply(self, x2, self.bias).reshape(*lead, -1)


class ColumnParallelLinear(LinearBase):
    def __init__(self, in_features, out_features, bias=False, dtype=torch.bfloat16, quant_method=None,
                 gather_output=False, prefix=""):
        super().__init__(in_features, out_features, bias, dtype, quant_method, prefix)
        self.tp = ps.tp_size()
        assert out_features % self.tp == 0
        self.gather_output = gather_output
        self._make(in_features, out_features // self.tp, bias)

    def weight_loader(self, param, loaded, shard_id=None):
        r = ps.tp_rank()
        out_dim = getattr(param, "output_dim", 0)
        n = param.shape[out_dim]
        loaded = _expand_scalar(param, loaded, self.out_features)
        param.data.copy_(loaded.narrow(out_dim, r * n, n))

    def forward(self, x):
        x2, lead = self._x2d(x)
        y = self.quant_method.apply(self, x2, self.bias)
        if self.gather_output and self.tp > 1:
            y = ps.tensor_model_parallel_all_gather(y, -1)
        return y.reshape(*lead, -1)


class MergedColumnParallelLinear(ColumnParallelLinear):
    """Several column-parallel projections of the same input fused in one weight (gate|up)."""

    def __init__(self, in_features, output_sizes: Sequence[int], bias=False, dtype=torch.bfloat16,
                 quant_method=None, prefix=""):
        self.output_sizes = list(output_sizes)
        super().__init__(in_features, sum(output_sizes), bias, dtype, quant_method, prefix=prefix)

    def weight_loader(self, param, loaded, shard_id=None):
        out_dim = getattr(param, "output_dim", 0)
        scale = getattr(param, "block_n", 1)  # block-scale tensors cover `block_n` output rows per entry
        loaded = _expand_scalar(param, loaded, sum(self.output_sizes) if shard_id is None else self.output_sizes[shard_id])
        if shard_id is None:  # already merged on disk
            per = [s // self.tp for s in self.output_sizes]
            off_src = off_dst = 0
            for s, p in zip(self.output_sizes, per):
                src = loaded.narrow(out_dim, (off_src + ps.tp_rank() * p) // scale, max(p // scale, 1))
                param.data.narrow(out_dim, off_dst // scale, max(p // scale, 1)).copy_(src)
                off_src += s
                off_dst += p
            return
        per = self.output_sizes[shard_id] // self.tp
        off = sum(self.output_sizes[:shard_id]) // self.tp
        src = loaded.narrow(out_dim, (ps.tp_rank() * per) // scale, max(per // scale, 1))
        param.data.narrow(out_dim, off // scale, max(per // scale, 1)).copy_(src)


class GateUpSiluLinear(LinearBase):
    """``silu(x W_gate^T) * (x W_up^T)`` as ONE tcgen05 GEMM with the activation in its epilogue.

    The (column-parallel) gate and up shards are stored row-interleaved - row ``2j`` is
    ``gate_j``, row ``2j+1`` is ``up_j`` - so every accumulator tile holds matching pairs.
    Unquantised weights only; quantised checkpoints use ``MergedColumnParallelLinear`` + the
    activation kernel.
    """

    def __init__(self, in_features: int, intermediate_size: int, dtype=torch.bfloat16, prefix: str = ""):
        super().__init__(in_features, 2 * intermediate_size, False, dtype, None, prefix)
        self.tp = ps.tp_size()
        assert intermediate_size % self.tp == 0
        self.inter_local = intermediate_size // self.tp
        self._make(in_features, 2 * self.inter_local, False)

    def weight_loader(self, param, loaded, shard_id=None):
        r, n = ps.tp_rank(), self.inter_local
        if shard_id is None:  # merged [gate; up] on disk
            full = loaded.shape[0] // 2
            self.weight_loader(param, loaded[:full], 0)
            self.weight_loader(param, loaded[full:], 1)
            return
        param.data[int(shard_id)::2].copy_(loaded.narrow(0, r * n, n))

    def forward(self, x):
        x2, lead = self._x2d(x)
        return ops.gemm_silu_mul(x2, self.weight).reshape(*lead, -1)


class QKVParallelLinear(ColumnParallelLinear):
    """Fused q/k/v projection; KV heads are replicated when there are fewer than TP ranks."""

    def __init__(self, hidden_size, head_size, total_num_heads, total_num_kv_heads, bias=False,
                 dtype=torch.bfloat16, quant_method=None, prefix=""):
        tp = ps.tp_size()
        self.head_size = head_size
        self.total_num_heads = total_num_heads
        self.total_num_kv_heads = total_num_kv_heads
        self.num_heads = total_num_heads // tp
        if total_num_kv_heads >= tp:
            self.num_kv_heads = total_num_kv_heads // tp
            self.kv_replicas = 1
        else:
            self.num_kv_heads = 1
            self.kv_replicas = tp // total_num_kv_heads
        out = (self.num_heads + 2 * self.num_kv_heads) * head_size * tp
        LinearBase.__init__(self, hidden_size, out, bias, dtype, quant_method, prefix)
        self.tp = tp
        self.gather_output = False
        self._make(hidden_size, (self.num_heads + 2 * self.num_kv_heads) * head_size, bias)

    def weight_loader(self, param, loaded, shard_id=None):
        out_dim = getattr(param, "output_dim", 0)
        scale = getattr(param, "block_n", 1)
        r = ps.tp_rank()
        q_sz = self.num_heads * self.head_size
        kv_sz = self.num_kv_heads * self.head_size
        offs = {"q": 0, "k": q_sz, "v": q_sz + kv_sz}
        sizes = {"q": q_sz, "k": kv_sz, "v": kv_sz}
        tq = self.total_num_heads * self.head_size
        tkv = self.total_num_kv_heads * self.head_size
        loaded = _expand_scalar(param, loaded, tq + 2 * tkv if shard_id is None else (tq if shard_id == "q" else tkv))
        if shard_id is None:
            for sid, src_off in (("q", 0), ("k", tq), ("v", tq + tkv)):
                tot = tq if sid == "q" else tkv
                self.weight_loader(param, loaded.narrow(out_dim, src_off // scale, max(tot // scale, 1)), sid)
            return
        shard_rank = r if shard_id == "q" else r // self.kv_replicas
        n = sizes[shard_id]
        src = loaded.narrow(out_dim, (shard_rank * n) // scale, max(n // scale, 1))
        param.data.narrow(out_dim, offs[shard_id] // scale, max(n // scale, 1)).copy_(src)


class RowParallelLinear(LinearBase):
    def __init__(self, in_features, out_features, bias=False, dtype=torch.bfloat16, quant_method=None,
                 reduce_results=True, input_is_parallel=True, prefix=""):
        super().__init__(in_features, out_features, bias, dtype, quant_method, prefix)
        self.tp = ps.tp_size()
        assert in_features % self.tp == 0
        self.reduce_results = reduce_results
        self.input_is_parallel = input_is_parallel
        self._make(in_features // self.tp, out_features, bias)

    def weight_loader(self, param, loaded, shard_id=None):
        in_dim = getattr(param, "input_dim", 1)
        loaded = _expand_scalar(param, loaded, self.out_features)
        if param.dim() <= in_dim or getattr(param, "expand_scalar", False):  # per-output-channel values are replicated
            param.data.copy_(loaded.reshape(param.shape))
            return
        n = param.shape[in_dim]
        param.data.copy_(loaded.narrow(in_dim, ps.tp_rank() * n, n))

    def forward(self, x, residual: Optional[torch.Tensor] = None):
        """``residual`` (rank 0 only adds it before the reduction) is folded into the GEMM epilogue."""
        x2, lead = self._x2d(x)
        bias = self.bias if (self.bias is not None and ps.tp_rank() == 0) else None
        res = residual if (residual is not None and (self.tp == 1 or ps.tp_rank() == 0)) else None
        y = self.quant_method.apply(self, x2, bias, res)
        if self.reduce_results and self.tp > 1:
            y = ps.tensor_model_parallel_all_reduce(y)
        return y.reshape(*lead, -1)
