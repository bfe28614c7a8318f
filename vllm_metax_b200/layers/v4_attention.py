"""DeepSeek-V4 attention: one shared 512-wide K = V vector per token, a sliding window of raw vectors and a
ratio-c compressed cache, an attention sink per head, a grouped low-rank output projection.

Per layer (``compress_ratio`` r from the checkpoint's ``compress_ratios``):

    r <= 1   window only: a query at position p attends the raw vectors of positions p - W + 1 .. p
    r = 128  + every complete compressed entry j < (p + 1) // r                     (dense)
    r = 4    + the ``index_topk`` compressed entries an indexer picks among them     (sparse)

Compression (``V4Compressor``): every token contributes a value row and a score row (a learned per-slot bias
``ape[p % r]`` is added to the score); entry j is the per-channel softmax(score)-weighted sum of the value rows of
block j - for r = 4 of blocks j - 1 and j, which use the first / second half of their 2 x 512 features - then
RMSNorm, interleaved-pair RoPE on the last 64 channels at position j * r, and a store into the compressed cache.
The softmax runs as an online accumulator ``(max, sum, weighted sum)`` per channel: a step reduces its tokens per
(request, block) segment, merges the partial accumulator carried from the request's previous step, emits an entry at
every block end and keeps at most three accumulators per request (18 KB) instead of the last 2r raw rows.  All
shapes depend only on the step's token count, so the same code runs under CUDA graphs.

Caches per layer, all paged by the request's block table: raw vectors ``[blocks, bs, 576]`` (512 used, the kernel's
row is 576 wide), compressed entries ``[blocks, bs / r, 576]``, index keys ``[blocks, (bs / r) * 132]`` bytes.  A
query token is handed to the latent-attention kernel as a request of its own, whose length is the number of entries it
may see: the window part runs the sparse kernel over W explicit positions, the compressed part the dense (r = 128)
or sparse (r = 4) kernel; both return log-sum-exps, which merge the two parts and apply the sink
``out *= sigmoid(lse - sink)``.

Parity: vllm_metax/models/deepseek_v4/attention.py:100-373 (projections, q norm + RoPE + cache insert, indexer
:380-552), compressor.py:25-128 (state write + compress / norm / RoPE / store), flashmla.py and
v1/attention/backends/mla/sparse_swa.py:152-616 (window + compressed index lists, sink), upstream's
``fused_inv_rope_fp8_quant`` + grouped einsum for the output side.
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.nn as nn

from .. import _custom_ops as ops
from ..attention.metadata import get_forward_context
from ..config import ModelConfig
from ..parallel import state as ps
from .basic import RMSNorm, get_rope
from .linear import ColumnParallelLinear, ReplicatedLinear, RowParallelLinear

NEG = -1.0e30          # "empty" running maximum (finite, so that differences never produce NaN)


# ----------------------------------------------------------------------------------------------- small helpers
def rope_tail(x: torch.Tensor, positions: torch.Tensor, cos_sin_cache: torch.Tensor, rope_dim: int,
              inverse: bool = False) -> torch.Tensor:
    """Interleaved-pair (GPT-J) rotation of the LAST ``rope_dim`` channels of ``x [T, ..., D]`` at ``positions [T]``;
    ``inverse`` rotates back.  Returns a new tensor in x's dtype (fp32 arithmetic)."""
    half = rope_dim // 2
    cs = cos_sin_cache.index_select(0, positions.long()).float()
    cos, sin = cs[:, :half], cs[:, half:]
    if inverse:
        sin = -sin
    shape = [x.shape[0]] + [1] * (x.dim() - 2) + [half]
    cos, sin = cos.view(shape), sin.view(shape)
    head, tail = x[..., : x.shape[-1] - rope_dim], x[..., x.shape[-1] - rope_dim:].float()
    a, b = tail[..., 0::2], tail[..., 1::2]
    rot = torch.stack([a * cos - b * sin, a * sin + b * cos], dim=-1).flatten(-2)
    return torch.cat([head, rot.to(x.dtype)], dim=-1)


def _merge(p, q):
    """Two online-softmax accumulators ``(m, l, a)`` -> one."""
    m = torch.maximum(p[0], q[0])
    sp, sq = torch.exp(p[0] - m), torch.exp(q[0] - m)
    return m, p[1] * sp + q[1] * sq, p[2] * sp + q[2] * sq


def _select(cond, p, q):
    c = cond[:, None]
    return tuple(torch.where(c, a, b) for a, b in zip(p, q))


def _segment_accumulate(score: torch.Tensor, value: torch.Tensor, seg_start: torch.Tensor):
    """Per-channel online softmax over the tokens of each segment (all tokens that share ``seg_start``); the result
    rows are valid at the segment-start rows and gathered back to every token of the segment."""
    T, D = score.shape
    idx = seg_start[:, None].expand(T, D)
    m = torch.full((T, D), NEG, dtype=torch.float32, device=score.device).scatter_reduce(0, idx, score, "amax")
    m_tok = m.index_select(0, seg_start)
    e = torch.exp(score - m_tok)
    l = torch.zeros(T, D, dtype=torch.float32, device=score.device).index_add_(0, seg_start, e)
    a = torch.zeros(T, D, dtype=torch.float32, device=score.device).index_add_(0, seg_start, e * value)
    return m_tok, l.index_select(0, seg_start), a.index_select(0, seg_start)


# ----------------------------------------------------------------------------------------------- compressor
class V4Compressor(nn.Module):
    """Turns the token stream into one compressed entry per ``ratio`` tokens (see the module docstring).

    ``forward`` returns ``(entry [T, head_dim], is_block_end [T], entry_index [T])``: row t holds the finished entry
    when token t closes a block, and is garbage otherwise (the caller stores rows under a -1 slot nowhere)."""

    def __init__(self, cfg: ModelConfig, head_dim: int, ratio: int, prefix: str):
        super().__init__()
        assert ratio > 1
        self.ratio, self.head_dim = ratio, head_dim
        self.coff = 2 if ratio == 4 else 1                  # ratio 4 pools over two overlapping blocks
        self.rope_dim = cfg.qk_rope_head_dim
        self.eps = cfg.rms_norm_eps
        self.ape = nn.Parameter(torch.zeros(ratio, self.coff * head_dim, dtype=torch.float32), requires_grad=False)
        # value rows | score rows, computed in fp32 by the reference (torch.mm(..., out_dtype=float32))
        self.fused_wkv_wgate = ReplicatedLinear(cfg.hidden_size, 2 * self.coff * head_dim, False, cfg.dtype,
                                                prefix=f"{prefix}.fused_wkv_wgate")
        self.norm = RMSNorm(head_dim, cfg.rms_norm_eps, cfg.dtype)
        self.state: Optional[torch.Tensor] = None

    def allocate_state(self, slots: int, device) -> int:
        """Per request: the partial accumulators of the open block (one per feature half) and, with overlapping blocks,
        the finished first-half accumulator of the previous block.  ``[slots, K, 3 (max, sum, weighted sum), D]``."""
        k = 3 if self.coff == 2 else 1
        self.state = torch.zeros(slots, k, 3, self.head_dim, dtype=torch.float32, device=device)
        self.state[:, :, 0] = NEG
        return self.state.numel() * 4

    def forward(self, x: torch.Tensor, positions: torch.Tensor, cos_sin_cache: torch.Tensor):
        md = get_forward_context().attn_metadata
        T, r, D, coff = x.shape[0], self.ratio, self.head_dim, self.coff
        dev = x.device
        if self.state is None:
            self.allocate_state(md.num_reqs + 1, dev)
        qsl = md.query_start_loc.long()
        B = qsl.numel() - 1
        slots = md.extra["state_indices"].long() if "state_indices" in md.extra else torch.arange(B, device=dev)
        tok = torch.arange(T, device=dev)
        req = torch.bucketize(tok, qsl[1:], right=True).clamp_max(B - 1)
        first_tok = qsl.index_select(0, req)
        pos = positions.long()
        chunk_start = pos - (tok - first_tok)                        # position of the request's first token in this step
        seg_start_pos = torch.maximum(pos - pos % r, chunk_start)
        seg_start = tok - (pos - seg_start_pos)                      # row of the first token of (request, block) here
        carries = (seg_start_pos % r) != 0                           # the block was opened by an earlier step
        block_end = (pos % r) == (r - 1)

        kv_score = self.fused_wkv_wgate(x).float()
        kv, score = kv_score[:, : coff * D], kv_score[:, coff * D:]
        score = score + self.ape.index_select(0, pos % r)
        slot_tok = slots.index_select(0, req)
        st = self.state

        def from_state(k):
            s = st[slot_tok, k]
            return s[:, 0], s[:, 1], s[:, 2]

        accs = []
        for f in range(coff):
            seg = _segment_accumulate(score[:, f * D:(f + 1) * D].contiguous(), kv[:, f * D:(f + 1) * D].contiguous(),
                                      seg_start)
            accs.append(_select(carries, _merge(from_state(f), seg), seg))
        if coff == 2:
            # window of block j = first-half features of block j - 1 and second-half features of block j
            t_prev = tok - r
            prev_here = tuple(a.index_select(0, t_prev.clamp_min(0)) for a in accs[0])
            prev = _select(t_prev >= first_tok, prev_here, from_state(2))
            empty = (torch.full_like(prev[0], NEG), torch.zeros_like(prev[1]), torch.zeros_like(prev[2]))
            win = _merge(_select(pos >= r, prev, empty), accs[1])
        else:
            win = accs[0]
        comp = win[2] / win[1].clamp_min(1e-30)

        # ---- carry: what the request's next step needs, taken at the request's last token of this step
        last = (qsl[1:] - 1).clamp_min(0)
        end_l = block_end.index_select(0, last)

        def rows(acc, at):
            return torch.stack([a.index_select(0, at) for a in acc], dim=1)          # [B, 3, D]

        blank = torch.zeros(B, 3, D, dtype=torch.float32, device=dev)
        blank[:, 0] = NEG
        for f in range(coff):
            st[slots, f] = torch.where(end_l[:, None, None], blank, rows(accs[f], last))
        if coff == 2:
            last_end = last - (pos.index_select(0, last) % r) - 1                  # row of the last block end before it
            seen = (last_end >= qsl[:-1]) & ~end_l
            keep = torch.where(seen[:, None, None], rows(accs[0], last_end.clamp_min(0)), st[slots, 2])
            st[slots, 2] = torch.where(end_l[:, None, None], rows(accs[0], last), keep)

        # ---- RMSNorm (fp32), RoPE on the last channels at the block's first position
        w = self.norm.weight.float()
        normed = comp * torch.rsqrt(comp.pow(2).mean(-1, keepdim=True) + self.eps) * w
        entry = rope_tail(normed.to(x.dtype), pos - pos % r, cos_sin_cache, self.rope_dim)
        return entry, block_end, pos // r


def naive_compress(kv_score: torch.Tensor, ape: torch.Tensor, ratio: int, head_dim: int) -> torch.Tensor:
    """The pooling step written out for one whole sequence ``kv_score [L, 2 * coff * D]`` (value rows | score rows):
    ``[L // ratio, D]`` pooled rows before norm and RoPE.  Test oracle; mirrors the gather + softmax + weighted sum of
    the reference's fused kernel (one program per block end, ``(1 + overlap) * ratio`` state rows)."""
    L = kv_score.shape[0]
    coff = 2 if ratio == 4 else 1
    D = head_dim
    kv, score = kv_score[:, : coff * D].float(), kv_score[:, coff * D:].float()
    score = score + ape[torch.arange(L) % ratio]
    out = []
    for j in range(L // ratio):
        p = (j + 1) * ratio - 1
        rows, feats = [], []
        for w in range(coff * ratio):
            q = p - coff * ratio + 1 + w
            if q < 0:
                continue
            off = D if (coff == 2 and w >= ratio) else 0
            rows.append(score[q, off: off + D])
            feats.append(kv[q, off: off + D])
        sm = torch.softmax(torch.stack(rows), dim=0)
        out.append((sm * torch.stack(feats)).sum(0))
    return torch.stack(out) if out else torch.zeros(0, D)


# ----------------------------------------------------------------------------------------------- indexer (ratio 4)
class V4Indexer(nn.Module):
    """Picks ``index_topk`` compressed entries per query token: index queries from the q low-rank stream, index keys
    from a compressor of its own (128 wide), logits ``sum_h w_h relu(q_h . k)``, top-k."""

    def __init__(self, cfg: ModelConfig, ratio: int, prefix: str):
        super().__init__()
        self.n_heads, self.head_dim, self.topk = cfg.index_n_heads, cfg.index_head_dim, cfg.index_topk
        self.rope_dim, self.ratio = cfg.qk_rope_head_dim, ratio
        self.wq_b = ReplicatedLinear(cfg.q_lora_rank, self.n_heads * self.head_dim, False, cfg.dtype,
                                     prefix=f"{prefix}.wq_b")
        self.weights_proj = ReplicatedLinear(cfg.hidden_size, self.n_heads, False, cfg.dtype,
                                             prefix=f"{prefix}.weights_proj")
        self.compressor = V4Compressor(cfg, self.head_dim, ratio, f"{prefix}.compressor")
        self.softmax_scale = self.head_dim ** -0.5

    def forward(self, x, qr, positions, cos_sin_cache, idx_cache, comp_slots, table_tok, n_entries, per_block: int,
                max_entries: int) -> torch.Tensor:
        T = x.shape[0]
        q = rope_tail(self.wq_b(qr).view(T, self.n_heads, self.head_dim), positions, cos_sin_cache, self.rope_dim)
        q_fp8, q_scale = ops.per_token_group_quant_fp8(q.reshape(T * self.n_heads, self.head_dim).contiguous(),
                                                       self.head_dim, ue8m0=True)
        weights = (self.weights_proj(x).float() * q_scale.view(T, self.n_heads) * self.softmax_scale
                   * self.n_heads ** -0.5)
        k, _, _ = self.compressor(x, positions, cos_sin_cache)
        ops.indexer_k_quant_and_cache(k.contiguous(), idx_cache, comp_slots, per_block)
        one_each = torch.arange(T + 1, dtype=torch.int32, device=x.device)
        idx = ops.indexer_topk(q_fp8.view(T, self.n_heads, self.head_dim), weights, idx_cache, table_tok,
                               n_entries.clamp_min(1), one_each, self.topk, per_block, max_seq_len=max_entries)
        return torch.where(idx < n_entries[:, None], idx, torch.full_like(idx, -1))


# ----------------------------------------------------------------------------------------------- attention
class DeepseekV4Attention(nn.Module):
    LATENT_ROW = 576          # row width of the latent-attention kernels (512 used here)

    def __init__(self, cfg: ModelConfig, layer_idx: int, prefix: str):
        super().__init__()
        tp = ps.tp_size()
        self.cfg, self.layer_idx = cfg, layer_idx
        abs_idx = int(prefix.rsplit(".", 2)[1]) if prefix.rsplit(".", 2)[1].isdigit() else layer_idx
        ratios = cfg.compress_ratios or []
        self.ratio = max(1, int(ratios[abs_idx])) if abs_idx < len(ratios) else 1
        self.head_dim = cfg.head_dim or 512
        assert self.head_dim == 512, "the latent-attention kernels are built for 512-wide vectors"
        self.rope_dim = cfg.qk_rope_head_dim
        self.heads = cfg.num_attention_heads // tp
        self.groups = cfg.o_groups // tp
        assert cfg.num_attention_heads % tp == 0 and cfg.o_groups % tp == 0 and self.heads % max(self.groups, 1) == 0
        self.o_lora = cfg.o_lora_rank
        self.window = int(cfg.sliding_window or 128)
        self.eps = cfg.rms_norm_eps
        self.scale = self.head_dim ** -0.5
        self.q_lora = cfg.q_lora_rank
        D = self.head_dim
        self.fused_wqa_wkv = ReplicatedLinear(cfg.hidden_size, self.q_lora + D, False, cfg.dtype,
                                              prefix=f"{prefix}.fused_wqa_wkv")
        self.q_norm = RMSNorm(self.q_lora, cfg.rms_norm_eps, cfg.dtype)
        self.kv_norm = RMSNorm(D, cfg.rms_norm_eps, cfg.dtype)
        self.wq_b = ColumnParallelLinear(self.q_lora, cfg.num_attention_heads * D, False, cfg.dtype,
                                         prefix=f"{prefix}.wq_b")
        per_group = cfg.num_attention_heads * D // cfg.o_groups
        self.wo_a = ColumnParallelLinear(per_group, cfg.o_groups * self.o_lora, False, cfg.dtype, prefix=f"{prefix}.wo_a")
        self.wo_b = RowParallelLinear(cfg.o_groups * self.o_lora, cfg.hidden_size, False, cfg.dtype,
                                      prefix=f"{prefix}.wo_b")
        # -inf = no sink; the loader fills this rank's heads
        self.attn_sink = nn.Parameter(torch.full((self.heads,), float("-inf"), dtype=torch.float32), requires_grad=False)
        self.rope = get_rope(self.rope_dim, self.rope_dim, cfg.max_position_embeddings, cfg.rope_theta, False,
                             cfg.rope_scaling)
        self.compressor = V4Compressor(cfg, D, self.ratio, f"{prefix}.compressor") if self.ratio > 1 else None
        self.indexer = V4Indexer(cfg, self.ratio, f"{prefix}.indexer") if (self.ratio == 4 and cfg.index_topk > 0) else None

    def weight_loader(self, param, loaded, shard_id=None):
        """``attn_sink`` is stored for all heads; every rank keeps its own."""
        r = ps.tp_rank()
        param.data.copy_(loaded.reshape(-1)[r * self.heads:(r + 1) * self.heads].to(param.dtype))

    # ---- caches and per-request state --------------------------------------------------------------------------
    def allocate_kv_cache(self, num_blocks: int, block_size: int, dtype, device) -> dict:
        d = {"swa": torch.zeros(num_blocks, block_size, self.LATENT_ROW, dtype=dtype, device=device), "comp": None,
             "idx": None}
        if self.ratio > 1:
            if block_size % self.ratio:
                raise ValueError(f"block_size {block_size} must be a multiple of the compress ratio {self.ratio}")
            per = block_size // self.ratio
            d["comp"] = torch.zeros(num_blocks, per, self.LATENT_ROW, dtype=dtype, device=device)
            if self.indexer is not None:
                d["idx"] = torch.zeros(num_blocks, per * (self.indexer.head_dim + 4), dtype=torch.uint8, device=device)
        return d

    def bytes_per_block(self, block_size: int, elem: int) -> int:
        n = block_size * self.LATENT_ROW * elem
        if self.ratio > 1:
            n += (block_size // self.ratio) * self.LATENT_ROW * elem
            if self.indexer is not None:
                n += (block_size // self.ratio) * (self.indexer.head_dim + 4)
        return n

    def allocate_state(self, slots: int, device) -> int:
        n = 0
        if self.compressor is not None:
            n += self.compressor.allocate_state(slots, device)
        if self.indexer is not None:
            n += self.indexer.compressor.allocate_state(slots, device)
        return n

    # ---- forward --------------------------------------------------------------------------------------------------
    def forward(self, positions: torch.Tensor, x: torch.Tensor) -> torch.Tensor:
        ctx = get_forward_context()
        md = ctx.attn_metadata
        caches = ctx.kv_caches[self.layer_idx]
        T, H, D, dev = x.shape[0], self.heads, self.head_dim, x.device
        cs = self.rope.cos_sin_cache
        qr_kv = self.fused_wqa_wkv(x)
        qr, kv = self.q_norm(qr_kv[:, : self.q_lora].contiguous()), self.kv_norm(qr_kv[:, self.q_lora:].contiguous())
        q = self.wq_b(qr).view(T, H, D).float()
        q = (q * torch.rsqrt(q.pow(2).mean(-1, keepdim=True) + self.eps)).to(x.dtype)      # per-head norm, no weight
        q = rope_tail(q, positions, cs, self.rope_dim)
        kv = rope_tail(kv, positions, cs, self.rope_dim)
        pad = kv.new_zeros(T, self.LATENT_ROW - D)
        ops.concat_and_cache_mla(kv, pad, caches["swa"], md.slot_mapping)

        # every token as a request of its own
        pos = positions.long()
        qsl = md.query_start_loc.long()
        tok = torch.arange(T, device=dev)
        req = torch.bucketize(tok, qsl[1:], right=True).clamp_max(qsl.numel() - 2)
        table_tok = md.block_table.index_select(0, req)
        q_lat = torch.nn.functional.pad(q, (0, self.LATENT_ROW - D)).contiguous()

        W = self.window
        win = pos[:, None] - (W - 1) + torch.arange(W, device=dev)[None, :]
        win = torch.where(win >= 0, win, torch.full_like(win, -1)).to(torch.int32)
        lse = torch.empty(H, T, dtype=torch.float32, device=dev)
        out = ops.mla_decode(q_lat, caches["swa"], table_tok, (pos + 1).to(torch.int32), self.scale, topk_indices=win,
                             lse_out=lse, max_seq_len=md.max_seq_len)
        if self.compressor is not None:
            r, bs = self.ratio, md.block_size
            per = bs // r
            entry, end, _ = self.compressor(x, positions, cs)
            sm = md.slot_mapping
            comp_slots = torch.where(end & (sm >= 0), (sm // bs) * per + (sm % bs) // r, torch.full_like(sm, -1))
            ops.concat_and_cache_mla(entry, pad, caches["comp"], comp_slots)
            n_c = ((pos + 1) // r).to(torch.int32)
            max_entries = md.max_seq_len // r + 1
            sel = None
            if self.indexer is not None:
                sel = self.indexer(x, qr, positions, cs, caches["idx"], comp_slots, table_tok, n_c, per, max_entries)
                none = (sel >= 0).sum(1) == 0
                self.last_selected = sel          # read by tests and debugging tools
            else:
                none = n_c == 0
            lse_c = torch.empty(H, T, dtype=torch.float32, device=dev)
            out_c = ops.mla_decode(q_lat, caches["comp"], table_tok, n_c.clamp_min(1), self.scale, topk_indices=sel,
                                   lse_out=lse_c, max_seq_len=max_entries)
            lse_c = torch.where(none[None, :], torch.full_like(lse_c, float("-inf")), lse_c)
            out_c = torch.where(none[:, None, None], torch.zeros_like(out_c), out_c)
            out, lse = ops.merge_attn_states(out, lse, out_c, lse_c, want_lse=True)
        # sink: one more softmax column that carries no value
        out = out.float() * torch.sigmoid(lse.t() - self.attn_sink[None, :])[..., None]
        out = rope_tail(out.to(x.dtype), positions, cs, self.rope_dim, inverse=True)
        G = self.groups
        z = torch.einsum("tgk,grk->tgr", out.reshape(T, G, (H // G) * D),
                         self.wo_a.weight.view(G, self.o_lora, (H // G) * D))
        return self.wo_b(z.reshape(T, G * self.o_lora))


def naive_v4_attention(q, kv_all, comp_all, pos: int, window: int, ratio: int, scale: float, sink, selected=None):
    """One query token written out: ``q [H, D]`` against the raw vectors ``kv_all [L, D]`` of its window and the
    compressed entries ``comp_all [n, D]`` that are complete at ``pos`` (or ``selected`` of them), with the sink column.
    Test oracle for ``DeepseekV4Attention``."""
    keys = [kv_all[max(0, pos - window + 1): pos + 1]]
    if ratio > 1:
        n = (pos + 1) // ratio
        ids = list(range(n)) if selected is None else [int(i) for i in selected if 0 <= int(i) < n]
        if ids:
            keys.append(comp_all[ids])
    k = torch.cat(keys).float()
    s = (q.float() @ k.t()) * scale                                    # [H, n_keys]
    s = torch.cat([s, sink.float()[:, None]], dim=1)
    p = torch.softmax(s, dim=-1)[:, :-1]
    return p @ k
