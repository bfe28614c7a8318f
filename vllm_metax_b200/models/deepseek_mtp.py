"""DeepSeek-V3 / V3.2 multi-token-prediction (MTP) module and the draft proposer built on it.

An MTP layer ``i`` predicts the token at offset ``i + 2`` from (a) the embedding of the token at offset
``i + 1`` and (b) the previous module's hidden state of the current position:

    x = eh_proj( [ enorm(embed(next_token)) | hnorm(prev_hidden) ] )  ->  one decoder block  ->  shared head

Checkpoint names (``model.layers.{L+i}.{enorm,hnorm,eh_proj,shared_head.norm,shared_head.head,embed_tokens}``
plus the block's ``self_attn`` / ``mlp`` / layernorms) map one-to-one onto this module tree; the per-layer
copy of ``embed_tokens`` is folded onto the shared embedding.

``MTPProposer`` runs the module after every target step over the same token rows (same attention metadata
and block tables, its own one-layer latent cache), so its KV cache follows the target's, and proposes the
arg-max token of the last valid row of every decoding request.

Parity: vllm_metax/models/deepseek_mtp.py (SharedHead, DeepSeekMultiTokenPredictorLayer,
DeepSeekMultiTokenPredictor, DeepSeekMTP.load_weights name rewriting).
"""
from __future__ import annotations

from typing import Iterable

import torch
import torch.nn as nn

from ..attention.metadata import ForwardContext, set_forward_context
from ..config import ModelConfig
from ..layers.basic import ParallelLMHead, RMSNorm, VocabParallelEmbedding
from ..layers.linear import ReplicatedLinear
from ..layers.mla import IndexerBackend, MLABackend
from .. import _custom_ops as ops
from .deepseek_v2 import DeepseekV2DecoderLayer, DeepseekV2ForCausalLM


class SharedHead(nn.Module):
    def __init__(self, cfg: ModelConfig):
        super().__init__()
        self.norm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps, cfg.dtype)
        self.head = ParallelLMHead(cfg.vocab_size, cfg.hidden_size, cfg.dtype)


class MultiTokenPredictorLayer(DeepseekV2DecoderLayer):
    """A decoder block (inherited: self_attn, mlp, layernorms) with the MTP input projection and head."""

    def __init__(self, cfg: ModelConfig, kv_index: int, prefix: str):
        super().__init__(cfg, kv_index, prefix)
        self.enorm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps, cfg.dtype)
        self.hnorm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps, cfg.dtype)
        self.eh_proj = ReplicatedLinear(2 * cfg.hidden_size, cfg.hidden_size, False, cfg.dtype, prefix=f"{prefix}.eh_proj")
        self.shared_head = SharedHead(cfg)

    def predict(self, embeds: torch.Tensor, positions: torch.Tensor, prev_hidden: torch.Tensor) -> torch.Tensor:
        # position 0 has no predecessor: its embedding input is masked, as in training
        e = self.enorm(embeds) * (positions > 0).to(embeds.dtype)[:, None]
        x = self.eh_proj(torch.cat([e, self.hnorm(prev_hidden)], dim=-1))
        h, residual = DeepseekV2DecoderLayer.forward(self, positions, x, None)
        return h + residual


class _MTPBody(nn.Module):
    def __init__(self, cfg: ModelConfig):
        super().__init__()
        L, n = cfg.num_hidden_layers, max(1, cfg.num_nextn_predict_layers)
        self.embed_tokens = VocabParallelEmbedding(cfg.vocab_size, cfg.hidden_size, cfg.dtype)
        self.layers = nn.ModuleDict({str(L + i): MultiTokenPredictorLayer(cfg, i, f"model.layers.{L + i}")
                                     for i in range(n)})
        self.first, self.count = L, n


class DeepSeekMTP(DeepseekV2ForCausalLM):
    """Architecture ``DeepSeekMTPModel``; reuses the base class' weight loading (expert stacking, fused
    ``q_a`` / ``kv_a`` projection, fp8 scales) after rewriting the MTP-specific names."""

    def __init__(self, cfg: ModelConfig):
        nn.Module.__init__(self)
        self.cfg = cfg
        self.model = _MTPBody(cfg)
        self.lm_head = None

    def num_kv_layers(self) -> int:
        return self.model.count

    def allocate_kv_cache(self, num_blocks, block_size, kv_cache_dtype, device):
        out = []
        for _ in range(self.model.count):
            d = {"mla": MLABackend.allocate(num_blocks, block_size, self.cfg.dtype, kv_cache_dtype, device), "idx": None}
            if self.cfg.has_indexer:
                d["idx"] = IndexerBackend.allocate(num_blocks, block_size, self.cfg.index_head_dim, device)
            out.append(d)
        return out

    def layer(self, spec_step_idx: int = 0) -> MultiTokenPredictorLayer:
        return self.model.layers[str(self.model.first + spec_step_idx % self.model.count)]

    def forward(self, input_ids, positions, hidden_states, spec_step_idx: int = 0):
        return self.layer(spec_step_idx).predict(self.model.embed_tokens(input_ids), positions, hidden_states)

    def compute_logits(self, hidden, spec_step_idx: int = 0):
        head = self.layer(spec_step_idx).shared_head
        return head.head.logits(head.norm(hidden))

    def load_weights(self, weights: Iterable[tuple[str, torch.Tensor]]) -> set[str]:
        first, last = self.model.first, self.model.first + self.model.count

        def rewrite():
            for name, w in weights:
                parts = name.split(".")
                if len(parts) < 4 or parts[:2] != ["model", "layers"] or not parts[2].isdigit():
                    continue
                if not (first <= int(parts[2]) < last):
                    continue                                  # a target-model layer
                if parts[3] == "embed_tokens":
                    yield "model.embed_tokens." + ".".join(parts[4:]), w
                else:
                    yield name, w

        return super().load_weights(rewrite())


class MTPProposer:
    """Draft proposer over a ``DeepSeekMTP`` module.  ``after_step`` is called by the engine once the target
    step's tokens are known."""

    def __init__(self, cfg, engine, architecture: str = "DeepSeekMTPModel", draft_model=None):
        """``architecture`` names the draft module class; ``draft_model`` (a ``ModelConfig``) replaces the copy of the
        target's configuration when the draft has its own (EAGLE heads)."""
        import copy

        from ..engine.loader import build_model

        self.k = 1
        self.engine = engine
        runner = engine.runner
        ecfg = copy.copy(engine.cfg)
        ecfg.model = copy.copy(draft_model if draft_model is not None else engine.cfg.model)
        ecfg.model.architecture = architecture
        self.module = build_model(ecfg, runner.device)
        if hasattr(self.module, "share_with_target") and not getattr(cfg, "own_embeddings", False):
            self.module.share_with_target(runner.model)
        self.kv_caches = self.module.allocate_kv_cache(runner.num_blocks, runner.block_size, ecfg.cache.kv_cache_dtype,
                                                       runner.device)
        runner.use_graphs = False          # the proposer needs the hidden states of every step
        runner.keep_hidden = True

    @torch.no_grad()
    def after_step(self, so, sampled: dict) -> None:
        runner = self.engine.runner
        last = getattr(runner, "last_step", None)
        if last is None:
            return
        h, md, T = last
        ids = runner.input_ids[:T].clone()
        # shift left inside every request's segment; the slot after the last fed token takes the step's new token
        # (or the next known token of a chunked prompt)
        rows, reqs = [], []
        t = 0
        nxt = torch.empty(T, dtype=torch.int64)
        host_ids = ids.cpu()
        for s in so.scheduled:
            r, n = s.request, s.num_new_tokens
            seg = host_ids[t:t + n]
            nxt[t:t + n - 1] = seg[1:]
            valid_last = t + n - 1
            pos_next = s.start_pos + n
            if s.num_spec:
                # only the accepted prefix is valid; the new token follows the last accepted row
                acc = len(r.output_token_ids) and (r.num_computed_tokens - s.start_pos - 1)
                valid_last = t + max(acc, 0)
                pos_next = s.start_pos + max(acc, 0) + 1
            nxt[valid_last] = r.token_at(pos_next) if pos_next < r.num_tokens else 0
            if not r.status.finished and r.output_token_ids and r.num_computed_tokens == r.num_tokens - 1:
                rows.append(valid_last)
                reqs.append(r)
            t += n
        ctx = ForwardContext(md, self.kv_caches, runner.positions[:T])
        with set_forward_context(ctx):
            hm = self.module(nxt.to(ids.device), runner.positions[:T], h)
        if not rows:
            return
        idx = torch.tensor(rows, device=hm.device)
        logits = self.module.compute_logits(hm.index_select(0, idx))
        out = torch.empty(len(rows), dtype=torch.int64, device=hm.device)
        toks = ops.argmax(logits, out).tolist()
        for r, tok in zip(reqs, toks):
            if r.params.max_tokens - len(r.output_token_ids) > 1:
                r.spec_token_ids = [int(tok)]
