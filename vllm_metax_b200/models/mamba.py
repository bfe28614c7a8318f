"""Mamba (selective state-space) decoder: no attention and no KV cache - every layer keeps a convolution carry and an
SSM state per running request in the runner's state slots.

    layer:  x, z = in_proj(RMSNorm(h))
            x    = silu(causal_conv1d(x))                      csrc/causal_conv1d.cu (carry [K-1, d_inner])
            dt, B, C = x_proj(x);  dt = dt_proj(dt)
            y    = selective_scan(x, softplus(dt + bias), -exp(A_log), B, C, D) * silu(z)     csrc/mamba_scan.cu
            h    = h + out_proj(y)

Single-rank (the mixer's projections are replicated).  Parity: the selective-scan kernel of the reference
(csrc/mamba/mamba_ssm/selective_scan_fwd.cu) and upstream's Mamba model that runs on it.
"""
from __future__ import annotations

from typing import Iterable, Optional

import torch
import torch.nn as nn

from ..attention.metadata import get_forward_context
from ..config import ModelConfig
from ..layers.basic import ParallelLMHead, RMSNorm, VocabParallelEmbedding
from ..layers.linear import ReplicatedLinear
from ..ops import gdn
from ..ops.extra import selective_scan_fwd
from ..parallel import state as ps


class MambaMixer(nn.Module):
    def __init__(self, cfg: ModelConfig):
        super().__init__()
        hf = cfg.hf_config
        self.d_inner = int(hf.get("intermediate_size") or hf.get("expand", 2) * cfg.hidden_size)
        self.n = int(hf.get("state_size", 16))
        self.K = int(hf.get("conv_kernel", 4))
        r = hf.get("time_step_rank", "auto")
        self.rank = -(-cfg.hidden_size // 16) if r == "auto" else int(r)
        bias, conv_bias = bool(hf.get("use_bias", False)), bool(hf.get("use_conv_bias", True))
        d, dt = self.d_inner, cfg.dtype
        self.in_proj = ReplicatedLinear(cfg.hidden_size, 2 * d, bias, dt)
        self.conv_weight = nn.Parameter(torch.zeros(d, self.K, dtype=dt), requires_grad=False)
        self.conv_bias = nn.Parameter(torch.zeros(d, dtype=dt), requires_grad=False) if conv_bias else None
        self.x_proj = ReplicatedLinear(d, self.rank + 2 * self.n, False, dt)
        self.dt_proj = ReplicatedLinear(self.rank, d, False, dt)
        self.dt_bias = nn.Parameter(torch.zeros(d, dtype=torch.float32), requires_grad=False)
        self.A_log = nn.Parameter(torch.zeros(d, self.n, dtype=torch.float32), requires_grad=False)
        self.D = nn.Parameter(torch.ones(d, dtype=torch.float32), requires_grad=False)
        self.out_proj = ReplicatedLinear(d, cfg.hidden_size, bias, dt)
        self.dtype = dt
        self.conv_state: Optional[torch.Tensor] = None
        self.ssm_state: Optional[torch.Tensor] = None

    def allocate_state(self, slots: int, device) -> int:
        self.conv_state = torch.zeros(slots, self.K - 1, self.d_inner, dtype=self.dtype, device=device)
        self.ssm_state = torch.zeros(slots, self.d_inner, self.n, dtype=torch.float32, device=device)
        return self.conv_state.numel() * self.conv_state.element_size() + self.ssm_state.numel() * 4

    def forward(self, h: torch.Tensor) -> torch.Tensor:
        md = get_forward_context().attn_metadata
        idx, init, qsl = md.extra["state_indices"], md.extra["state_has_init"], md.query_start_loc
        xz = self.in_proj(h)
        x, z = xz[:, : self.d_inner], xz[:, self.d_inner:]
        x = gdn.causal_conv1d(x, self.conv_weight, self.conv_bias, self.conv_state, qsl, idx, init, silu=True)
        dbc = self.x_proj(x)
        dt = self.dt_proj(dbc[:, : self.rank].contiguous())
        B = dbc[:, self.rank: self.rank + self.n].t().unsqueeze(0).contiguous()            # [1, n, T]
        C = dbc[:, self.rank + self.n:].t().unsqueeze(0).contiguous()
        y, _ = selective_scan_fwd(x.t().contiguous(), dt.t().contiguous(), -torch.exp(self.A_log), B, C, self.D,
                                  z.t().contiguous(), self.dt_bias, True, self.ssm_state, qsl, idx, init)
        return self.out_proj(y.t().contiguous())


class MambaBlock(nn.Module):
    def __init__(self, cfg: ModelConfig):
        super().__init__()
        self.norm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps, cfg.dtype)
        self.mixer = MambaMixer(cfg)

    def forward(self, h):
        return h + self.mixer(self.norm(h))


class MambaForCausalLM(nn.Module):
    supports_prefix_caching = False
    renames = [(r"^backbone\.embeddings\.", "embeddings."), (r"^backbone\.layers\.", "layers."),
               (r"^backbone\.norm_f\.", "norm_f."), (r"\.mixer\.conv1d\.weight$", ".mixer.conv_weight"),
               (r"\.mixer\.conv1d\.bias$", ".mixer.conv_bias"), (r"\.mixer\.dt_proj\.bias$", ".mixer.dt_bias")]

    def __init__(self, cfg: ModelConfig):
        super().__init__()
        assert ps.tp_size() == 1 and ps.get_pp_group().world_size == 1, "Mamba runs on one rank"
        self.cfg = cfg
        cfg.tie_word_embeddings = cfg.hf_config.get("tie_word_embeddings", True)
        self.embeddings = VocabParallelEmbedding(cfg.vocab_size, cfg.hidden_size, cfg.dtype)
        self.layers = nn.ModuleList([MambaBlock(cfg) for _ in range(cfg.num_hidden_layers)])
        self.norm_f = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps, cfg.dtype)
        if cfg.tie_word_embeddings:
            self.lm_head = self.embeddings
            self.lm_head.__class__ = ParallelLMHead
        else:
            self.lm_head = ParallelLMHead(cfg.vocab_size, cfg.hidden_size, cfg.dtype)

    # ---- engine interface ------------------------------------------------------------
    def num_kv_layers(self) -> int:
        return 0

    def kv_cache_spec(self) -> dict:
        return {"kind": "gqa", "num_kv_heads": 1, "head_size": 64}       # no layer owns paged KV; blocks only meter length

    def allocate_state(self, slots: int, device) -> int:
        return sum(l.mixer.allocate_state(slots, device) for l in self.layers)

    def forward(self, input_ids, positions, intermediate=None):
        h = self.embeddings(input_ids)
        for layer in self.layers:
            h = layer(h)
        return self.norm_f(h)

    def compute_logits(self, hidden):
        return self.lm_head.logits(hidden)

    def load_weights(self, weights: Iterable[tuple[str, torch.Tensor]]) -> set[str]:
        import re

        params = dict(self.named_parameters())
        modules = dict(self.named_modules())
        loaded: set[str] = set()
        for name, w in weights:
            for pat, rep in self.renames:
                name = re.sub(pat, rep, name)
            if name.startswith("lm_head.") and self.cfg.tie_word_embeddings:
                continue
            if name not in params:
                continue
            p = params[name]
            if name.endswith("conv_weight"):
                w = w.reshape(w.shape[0], w.shape[-1])
            loader = getattr(modules[name.rsplit(".", 1)[0]], "weight_loader", None)
            if loader is not None and name.rsplit(".", 1)[1] in ("weight", "bias"):
                loader(p, w, None)
            else:
                p.data.copy_(w.reshape(p.shape).to(p.dtype))
            loaded.add(name)
        return loaded
