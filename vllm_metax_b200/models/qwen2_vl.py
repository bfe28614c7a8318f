"""Qwen2-VL: dynamic-resolution vision transformer + Qwen2 decoder with multimodal rotary positions (M-RoPE).

Vision side (``Qwen2VisionTower``): the processor hands over flattened patches ``[N, 3 * 2 * 14 * 14]`` and one
``(t, h, w)`` grid per image.  Patch embedding (the 3-D convolution is a linear map on a flattened patch), 2-D rotary
positions (half of each head's rotary pairs turn with the patch row, half with its column; rows / columns are numbered
in 2 x 2 merge-unit order, which is the order the patches arrive in), ``depth`` pre-LayerNorm blocks whose attention is
bidirectional inside one temporal frame (varlen, non-causal), and the merger that concatenates every 2 x 2 unit and
projects it to the decoder width: ``t * h * w / 4`` tokens per image.

Decoder side: the rotary angle of frequency pair ``j`` is taken from one of THREE position streams (temporal, height,
width) according to ``mrope_section`` - text tokens carry the same value in all three, image tokens their grid
coordinates, and the text after an image continues from the largest coordinate used.  The engine keeps ordinary 1-D
positions for the cache; the three streams travel as ``extra["mrope_positions"]`` (built per step by the model runner
from the request's prompt table and its offset for generated tokens) and ``LlamaAttention`` applies them.

Parity: Qwen2-VL / Qwen2.5-VL / Qwen3-VL rows of the reference's multimodal table (docs/models/supported_models.md:86-91),
its ``MRotaryEmbedding`` registration (registry/custom_ops/layers/rotary_embedding/rotary_embedding.py:9-32) and ViT
attention layer (registry/custom_ops/layers/attention/mm_encoder_attention.py:17-122).  Checked against Hugging Face's
``Qwen2VLForConditionalGeneration`` in ``tests/test_multimodal.py``.
"""
from __future__ import annotations

import hashlib
import re
from typing import Iterable, Optional

import numpy as np
import torch
import torch.nn as nn
import torch.nn.functional as F

from .. import _custom_ops as ops
from ..config import ModelConfig
from ..layers.basic import LayerNorm
from ..layers.linear import ReplicatedLinear
from ..layers.mm_encoder_attention import encoder_attention


def mrope_stream_of_frequency(sections, half: int, interleaved: bool) -> list:
    """Which of the three position streams (0 = temporal, 1 = height, 2 = width) turns frequency pair j.  Chunked
    (Qwen2-VL): the first ``sections[0]`` pairs are temporal, the next height, the rest width.  Interleaved
    (Qwen3-VL): pairs 1, 4, 7, ... below ``3 * sections[1]`` are height, pairs 2, 5, 8, ... below ``3 * sections[2]``
    width, everything else temporal."""
    if not interleaved:
        out = [0] * sections[0] + [1] * sections[1] + [2] * sections[2]
        assert len(out) == half, "mrope_section must cover half of the head dimension"
        return out
    out = [0] * half
    for j in range(half):
        if j % 3 == 1 and j < 3 * sections[1]:
            out[j] = 1
        elif j % 3 == 2 and j < 3 * sections[2]:
            out[j] = 2
    return out


def apply_mrope(q: torch.Tensor, k: torch.Tensor, pos3: torch.Tensor, cos_sin_cache: torch.Tensor, sections,
                head_dim: int, interleaved: bool = False, is_neox: bool = True) -> tuple[torch.Tensor, torch.Tensor]:
    """Rotation of ``q [T, Hq * D]`` / ``k [T, Hkv * D]`` where frequency pair j turns with the position stream
    ``mrope_stream_of_frequency`` names, taken from ``pos3 [3, T]``.  ``cos_sin_cache [max_pos, R]`` =
    ``[cos(R/2) | sin(R/2)]`` with ``R <= D`` rotated dimensions (the rest of a head passes through); pairs are
    (j, j + R/2) in NeoX style and (2j, 2j + 1) otherwise."""
    rot = cos_sin_cache.shape[1]
    half = rot // 2
    cs = cos_sin_cache.index_select(0, pos3.reshape(-1).long()).view(3, -1, rot).float()           # [3, T, R]
    sel = torch.as_tensor(mrope_stream_of_frequency(list(sections), half, interleaved), device=cs.device)
    j = torch.arange(half, device=cs.device)
    cos = cs[sel, :, j].transpose(0, 1)[:, None, :]                                               # [T, 1, R/2]
    sin = cs[sel, :, half + j].transpose(0, 1)[:, None, :]

    def turn(x):
        T = x.shape[0]
        x3 = x.reshape(T, -1, head_dim).float()
        xr, rest = x3[..., :rot], x3[..., rot:]
        if is_neox:
            a, b = xr[..., :half], xr[..., half:]
            out = torch.cat([a * cos - b * sin, b * cos + a * sin], -1)
        else:
            a, b = xr[..., 0::2], xr[..., 1::2]
            out = torch.stack([a * cos - b * sin, b * cos + a * sin], -1).flatten(-2)
        return torch.cat([out, rest], -1).to(x.dtype).reshape(T, -1)

    return turn(q), turn(k)


def mrope_prompt_positions(ids: list, grids, image_token_id: int, merge: int, video_token_id: Optional[int] = None,
                           video_grids: Optional[list] = None, video_t_scale: Optional[list] = None) -> tuple[np.ndarray, int]:
    """``[3, len(ids)]`` position streams of a prompt whose images (in order) have the ``(t, h, w)`` patch grids
    ``grids`` (and whose videos, runs of ``video_token_id``, have ``video_grids``), and the offset that turns the
    ordinary position of a generated token into its (common) stream value.  ``video_t_scale[i]``: how far the
    temporal stream advances per temporal patch of video i (1 = one step, as for Qwen2-VL; Qwen2.5-VL uses seconds per
    patch x position steps per second)."""
    pos = np.zeros((3, len(ids)), dtype=np.int64)
    queues = {image_token_id: [(g, 1.0) for g in grids]}
    if video_token_id is not None:
        scales = list(video_t_scale or [1.0] * len(video_grids or []))
        queues[video_token_id] = list(zip(video_grids or [], scales))
    nxt, i = 0, 0
    while i < len(ids):
        q = queues.get(ids[i])
        if q:
            (t, h, w), scale = q.pop(0)
            gh, gw = h // merge, w // merge
            n = t * gh * gw
            steps = np.floor(np.arange(t) * scale).astype(np.int64)
            tt = np.repeat(steps, gh * gw)
            hh = np.tile(np.repeat(np.arange(gh), gw), t)
            ww = np.tile(np.arange(gw), t * gh)
            pos[:, i:i + n] = np.stack([tt, hh, ww]) + nxt
            nxt += int(max(steps[-1], gh - 1, gw - 1)) + 1
            i += n
        else:
            pos[:, i] = nxt
            nxt += 1
            i += 1
    return pos, nxt - len(ids)


class Qwen2VisionBlock(nn.Module):
    def __init__(self, dim: int, heads: int, mlp_dim: int, act: str, dtype):
        super().__init__()
        self.heads, self.hd = heads, dim // heads
        self.norm1, self.norm2 = LayerNorm(dim, 1e-6, dtype), LayerNorm(dim, 1e-6, dtype)
        self.qkv = ReplicatedLinear(dim, 3 * dim, True, dtype)
        self.proj = ReplicatedLinear(dim, dim, True, dtype)
        self.fc1, self.fc2 = ReplicatedLinear(dim, mlp_dim, True, dtype), ReplicatedLinear(mlp_dim, dim, True, dtype)
        self.act = {"quick_gelu": "gelu_quick", "gelu": "gelu", "gelu_pytorch_tanh": "gelu_tanh"}.get(act, act)

    def forward(self, x, cos, sin, cu, max_tokens: int):
        N, dim = x.shape
        qkv = self.qkv(self.norm1(x)).reshape(N, 3, self.heads, self.hd)
        q, k, v = qkv[:, 0], qkv[:, 1], qkv[:, 2]

        def rot(t):      # rotate-half over the whole head, angles [N, hd] = [row | col | row | col] quarters
            tf_ = t.float()
            a, b = tf_[..., : self.hd // 2], tf_[..., self.hd // 2:]
            return (tf_ * cos[:, None, :] + torch.cat([-b, a], -1) * sin[:, None, :]).to(t.dtype)

        a = encoder_attention(rot(q).contiguous(), rot(k).contiguous(), v.contiguous(), cu, max_tokens)
        x = x + self.proj(a.reshape(N, dim))
        return x + self.fc2(ops.activation(self.fc1(self.norm2(x)), self.act))


class Qwen2VisionTower(nn.Module):
    def __init__(self, vc: dict, dtype):
        super().__init__()
        self.embed, self.heads = vc["embed_dim"], vc["num_heads"]
        self.patch, self.merge, self.tpatch = vc.get("patch_size", 14), vc.get("spatial_merge_size", 2), vc.get("temporal_patch_size", 2)
        self.in_ch = vc.get("in_channels", 3)
        self.patch_dim = self.in_ch * self.tpatch * self.patch * self.patch
        self.patch_embed = ReplicatedLinear(self.patch_dim, self.embed, False, dtype)
        mlp_dim = int(self.embed * vc.get("mlp_ratio", 4))
        self.blocks = nn.ModuleList([Qwen2VisionBlock(self.embed, self.heads, mlp_dim, vc.get("hidden_act", "quick_gelu"), dtype)
                                     for _ in range(vc["depth"])])
        unit = self.embed * self.merge * self.merge
        self.ln_q = LayerNorm(self.embed, 1e-6, dtype)
        self.merger_fc1 = ReplicatedLinear(unit, unit, True, dtype)
        self.merger_fc2 = ReplicatedLinear(unit, vc["hidden_size"], True, dtype)

    def _angles(self, grids: list, device) -> torch.Tensor:
        """``[N, head_dim / 2]``: per patch the angles of its row then of its column (quarter of the head each)."""
        hd = self.embed // self.heads
        dim = hd // 2
        inv = 1.0 / (10000.0 ** (torch.arange(0, dim, 2, dtype=torch.float32, device=device) / dim))
        m = self.merge
        out = []
        for t, h, w in grids:
            hp = torch.arange(h, device=device)[:, None].expand(h, w).reshape(h // m, m, w // m, m).permute(0, 2, 1, 3).flatten()
            wp = torch.arange(w, device=device)[None, :].expand(h, w).reshape(h // m, m, w // m, m).permute(0, 2, 1, 3).flatten()
            ang = torch.cat([hp[:, None].float() * inv[None, :], wp[:, None].float() * inv[None, :]], -1)
            out.append(ang.repeat(t, 1))
        return torch.cat(out)

    def forward(self, patches: torch.Tensor, grids: list) -> torch.Tensor:
        """``patches [N, patch_dim]`` -> ``[N / merge^2, hidden_text]``."""
        x = self.patch_embed(patches.to(self.patch_embed.weight.dtype))
        ang = self._angles(grids, x.device)
        emb = torch.cat([ang, ang], -1)
        cos, sin = emb.cos(), emb.sin()
        frames = [h * w for t, h, w in grids for _ in range(t)]
        cu = torch.tensor([0] + list(np.cumsum(frames)), dtype=torch.int32, device=x.device)
        for blk in self.blocks:
            x = blk(x, cos, sin, cu, max(frames))
        x = self.ln_q(x).reshape(-1, self.embed * self.merge * self.merge)
        return self.merger_fc2(F.gelu(self.merger_fc1(x)))


class Qwen2VLForConditionalGeneration(nn.Module):
    is_multimodal = True
    uses_mrope = True
    supports_video = True         # Qwen2-VL's video positions advance one step per temporal patch, like its images

    @property
    def video_token_id(self) -> int:
        return int(self.cfg.hf_config.get("video_token_id", 151656))
    image_mean, image_std = (0.48145466, 0.4578275, 0.40821073), (0.26862954, 0.26130258, 0.27577711)    # CLIP statistics
    renames = [(r"^model\.language_model\.", "language_model.model."), (r"^model\.visual\.", "visual."),
               (r"^lm_head\.", "language_model.lm_head."), (r"^model\.(?!language_model|visual)", "language_model.model."),
               (r"^visual\.patch_embed\.proj\.", "visual.patch_embed."),
               (r"^visual\.blocks\.(\d+)\.attn\.", r"visual.blocks.\1."), (r"^visual\.blocks\.(\d+)\.mlp\.", r"visual.blocks.\1."),
               (r"^visual\.merger\.ln_q\.", "visual.ln_q."), (r"^visual\.merger\.mlp\.0\.", "visual.merger_fc1."),
               (r"^visual\.merger\.mlp\.2\.", "visual.merger_fc2.")]

    def __init__(self, cfg: ModelConfig):
        super().__init__()
        from . import get_model_class

        self.cfg = cfg
        hf = cfg.hf_config
        self.image_token_id = int(hf.get("image_token_id", 151655))
        self.visual = Qwen2VisionTower(hf["vision_config"], cfg.dtype)
        self.language_model = get_model_class("Qwen2ForCausalLM")(cfg)
        tc = hf.get("text_config", hf)
        rp = tc.get("rope_parameters") or tc.get("rope_scaling") or hf.get("rope_scaling") or {}
        self.mrope_section = list(rp.get("mrope_section") or [cfg.head_dim // 2 - 2 * (cfg.head_dim // 6)] + [cfg.head_dim // 6] * 2)
        for layer in self.language_model.model.layers.values():
            layer.self_attn.mrope_section = self.mrope_section

    # ---- multimodal interface -------------------------------------------------------------------------------------
    def patchify(self, image) -> tuple[torch.Tensor, tuple]:
        """A PIL image / ``[3, H, W]`` tensor -> ``(patches [N, patch_dim], (1, h, w))``: resized so that both sides
        are multiples of ``patch * merge``, CLIP-normalised, one frame repeated over the temporal patch."""
        v = self.visual
        if not isinstance(image, torch.Tensor):
            image = torch.from_numpy(np.asarray(image.convert("RGB"))).permute(2, 0, 1)
        x = image.float() / (255.0 if image.dtype == torch.uint8 else 1.0)
        unit = v.patch * v.merge
        H = max(unit, round(x.shape[1] / unit) * unit)
        W = max(unit, round(x.shape[2] / unit) * unit)
        x = F.interpolate(x[None], size=(H, W), mode="bicubic", align_corners=False)[0].clamp(0, 1)
        mean, std = torch.tensor(self.image_mean).view(3, 1, 1), torch.tensor(self.image_std).view(3, 1, 1)
        x = ((x - mean) / std)[None].repeat(v.tpatch, 1, 1, 1)                       # [tp, 3, H, W]
        gh, gw, m, p = H // v.patch, W // v.patch, v.merge, v.patch
        x = x.reshape(1, v.tpatch, 3, gh // m, m, p, gw // m, m, p).permute(0, 3, 6, 4, 7, 2, 1, 5, 8)
        return x.reshape(gh * gw, 3 * v.tpatch * p * p), (1, gh, gw)

    @torch.no_grad()
    def encode_request(self, prompt_token_ids: list, mm: dict, device):
        """Everything the engine needs for one request: the prompt with its placeholder runs expanded, the projected
        image (and video) features with the prompt positions they replace, a content hash, and the M-RoPE streams of
        the prompt.  Videos come pre-processed: ``pixel_values_videos`` + ``video_grid_thw`` (``t`` temporal patches per
        video), their placeholder is the model's video token."""
        if "pixel_values" in mm:
            patches, grids = mm["pixel_values"], [tuple(int(x) for x in g) for g in mm["image_grid_thw"]]
        elif "image" in mm:
            imgs = mm["image"] if isinstance(mm["image"], (list, tuple)) else [mm["image"]]
            pg = [self.patchify(im) for im in imgs]
            patches, grids = torch.cat([p for p, _ in pg]), [g for _, g in pg]
        else:
            patches, grids = None, []
        vpatches, vgrids = mm.get("pixel_values_videos"), [tuple(int(x) for x in g) for g in mm.get("video_grid_thw", [])]
        vtok = self.video_token_id if vgrids else None
        if vgrids and not self.supports_video:
            raise ValueError(f"{type(self).__name__} takes images only")
        m2 = self.visual.merge ** 2
        tok = self.image_token_id
        kinds = {tok: (patches, grids)}
        if vtok is not None:
            kinds[vtok] = (vpatches, vgrids)
        feats_by, per_by = {}, {}
        for t_id, (px, gr) in kinds.items():
            if gr:
                feats_by[t_id] = self.visual(px.to(device), gr)
                per_by[t_id] = [t * h * w // m2 for t, h, w in gr]
            else:
                feats_by[t_id], per_by[t_id] = None, []
        # expand single placeholders / check the expanded runs, for either kind of token
        ids, used = [], {k: 0 for k in kinds}
        i, n_ids = 0, len(prompt_token_ids)
        while i < n_ids:
            t_id = prompt_token_ids[i]
            if t_id in kinds:
                j = i
                while j < n_ids and prompt_token_ids[j] == t_id:
                    j += 1
                run = j - i
                k = used[t_id]
                per = per_by[t_id]
                total, kk = 0, k
                while kk < len(per) and total < run:                   # expanded items back to back (usually one)
                    total += per[kk]
                    kk += 1
                if total == run:
                    ids.extend([t_id] * run)
                    used[t_id] = kk
                elif k + run <= len(per):                              # `run` single placeholders: expand each
                    for r in range(run):
                        ids.extend([t_id] * per[k + r])
                    used[t_id] += run
                else:
                    raise ValueError(f"prompt has a placeholder run of {run} tokens; the inputs need {per[k:]}")
                i = j
            else:
                ids.append(t_id)
                i += 1
        for t_id, per in per_by.items():
            if used[t_id] != len(per):
                raise ValueError(f"prompt has placeholders for {used[t_id]} of {len(per)} visual inputs")
        # features in prompt order
        arr = np.asarray(ids)
        pos = np.nonzero(np.isin(arr, list(kinds)))[0].astype(np.int64)
        if vtok is None:
            feats = feats_by[tok]
        else:
            width = next(f.shape[1] for f in feats_by.values() if f is not None)
            feats = torch.empty(len(pos), width, dtype=next(f.dtype for f in feats_by.values() if f is not None), device=device)
            for t_id, f in feats_by.items():
                if f is not None:
                    feats[torch.from_numpy(arr[pos] == t_id).to(device)] = f
        h = hashlib.sha256()
        for px in (patches, vpatches):
            if px is not None:
                h.update(px.detach().float().cpu().numpy().tobytes())
        table, delta = mrope_prompt_positions(ids, grids, tok, self.visual.merge, vtok, vgrids,
                                              self.video_t_scale(mm, len(vgrids)) if vgrids else None)
        return ids, (feats, pos, h.hexdigest()[:16]), {"mrope_positions": table, "mrope_delta": delta}

    def video_t_scale(self, mm: dict, n: int) -> list:
        """Temporal-stream advance per temporal patch of each video."""
        return [1.0] * n

    # ---- engine interface: the text decoder's ---------------------------------------------------------------------
    def num_kv_layers(self) -> int:
        return self.language_model.num_kv_layers()

    def kv_cache_spec(self) -> dict:
        return self.language_model.kv_cache_spec()

    def forward(self, input_ids, positions, intermediate=None):
        return self.language_model(input_ids, positions, intermediate)

    def compute_logits(self, hidden):
        return self.language_model.compute_logits(hidden)

    @property
    def model(self):
        return self.language_model.model

    def load_weights(self, weights: Iterable[tuple[str, torch.Tensor]]) -> set[str]:
        params = dict(self.named_parameters())
        text, loaded = [], set()
        for name, w in weights:
            for pat, rep in self.renames:
                name = re.sub(pat, rep, name)
            if name.startswith("language_model."):
                text.append((name[len("language_model."):], w))
                continue
            if name == "visual.patch_embed.weight":
                w = w.reshape(w.shape[0], -1)                # Conv3d kernel [embed, 3, tp, p, p] -> linear
            if name in params:
                params[name].data.copy_(w.reshape(params[name].shape))
                loaded.add(name)
        loaded |= {"language_model." + n for n in self.language_model.load_weights(iter(text))}
        return loaded


# ------------------------------------------------------------------------------------------------ Qwen2.5-VL
class Qwen25VisionBlock(nn.Module):
    """RMSNorm, attention, SiLU-gated MLP (all linears with bias)."""

    def __init__(self, dim: int, heads: int, inter: int, dtype):
        super().__init__()
        from ..layers.basic import RMSNorm

        self.heads, self.hd = heads, dim // heads
        self.norm1, self.norm2 = RMSNorm(dim, 1e-6, dtype), RMSNorm(dim, 1e-6, dtype)
        self.qkv = ReplicatedLinear(dim, 3 * dim, True, dtype)
        self.proj = ReplicatedLinear(dim, dim, True, dtype)
        self.gate_proj = ReplicatedLinear(dim, inter, True, dtype)
        self.up_proj = ReplicatedLinear(dim, inter, True, dtype)
        self.down_proj = ReplicatedLinear(inter, dim, True, dtype)

    def forward(self, x, cos, sin, cu, max_tokens: int):
        N, dim = x.shape
        qkv = self.qkv(self.norm1(x)).reshape(N, 3, self.heads, self.hd)

        def rot(t):
            tf_ = t.float()
            a, b = tf_[..., : self.hd // 2], tf_[..., self.hd // 2:]
            return (tf_ * cos[:, None, :] + torch.cat([-b, a], -1) * sin[:, None, :]).to(t.dtype)

        a = encoder_attention(rot(qkv[:, 0]).contiguous(), rot(qkv[:, 1]).contiguous(), qkv[:, 2].contiguous(), cu, max_tokens)
        x = x + self.proj(a.reshape(N, dim))
        h = self.norm2(x)
        return x + self.down_proj(F.silu(self.gate_proj(h)) * self.up_proj(h))


class Qwen25VisionTower(Qwen2VisionTower):
    """Qwen2.5-VL tower: most blocks attend inside windows of ``window_size`` pixels (merge units are reordered window
    by window, the order is undone after the merger); the blocks listed in ``fullatt_block_indexes`` attend the frame."""

    def __init__(self, vc: dict, dtype):
        nn.Module.__init__(self)
        from ..layers.basic import RMSNorm

        self.embed, self.heads = vc["hidden_size"], vc["num_heads"]
        self.patch, self.merge, self.tpatch = vc.get("patch_size", 14), vc.get("spatial_merge_size", 2), vc.get("temporal_patch_size", 2)
        self.in_ch = vc.get("in_channels", vc.get("in_chans", 3))
        self.patch_dim = self.in_ch * self.tpatch * self.patch * self.patch
        self.window = vc.get("window_size", 112) // self.merge // self.patch          # merge units per window side
        self.full_blocks = set(vc.get("fullatt_block_indexes", [7, 15, 23, 31]))
        self.patch_embed = ReplicatedLinear(self.patch_dim, self.embed, False, dtype)
        self.blocks = nn.ModuleList([Qwen25VisionBlock(self.embed, self.heads, vc["intermediate_size"], dtype)
                                     for _ in range(vc["depth"])])
        unit = self.embed * self.merge * self.merge
        self.ln_q = RMSNorm(self.embed, 1e-6, dtype)
        self.merger_fc1 = ReplicatedLinear(unit, unit, True, dtype)
        self.merger_fc2 = ReplicatedLinear(unit, vc["out_hidden_size"], True, dtype)

    def _windows(self, grids: list):
        """Order of the merge units window by window, and the cumulative patch counts of the windows."""
        order, cu, base, ws, m2 = [], [0], 0, self.window, self.merge * self.merge
        for t, h, w in grids:
            gh, gw = h // self.merge, w // self.merge
            idx = torch.arange(t * gh * gw).reshape(t, gh, gw)
            ph, pw = (ws - gh % ws) % ws, (ws - gw % ws) % ws
            idx = F.pad(idx, (0, pw, 0, ph), value=-100)
            nh, nw = (gh + ph) // ws, (gw + pw) // ws
            idx = idx.reshape(t, nh, ws, nw, ws).permute(0, 1, 3, 2, 4).reshape(t, nh * nw, ws, ws)
            lens = (idx != -100).sum([2, 3]).reshape(-1)
            order.append(idx[idx != -100] + base)
            for n in lens.tolist():
                if n:
                    cu.append(cu[-1] + n * m2)
            base += t * gh * gw
        return torch.cat(order), cu

    def forward(self, patches: torch.Tensor, grids: list) -> torch.Tensor:
        x = self.patch_embed(patches.to(self.patch_embed.weight.dtype))
        dev = x.device
        ang = self._angles(grids, dev)
        order, cu_win = self._windows(grids)
        order = order.to(dev)
        m2 = self.merge * self.merge
        N = x.shape[0]
        x = x.reshape(N // m2, m2, -1)[order].reshape(N, -1)
        ang = ang.reshape(N // m2, m2, -1)[order].reshape(N, -1)
        emb = torch.cat([ang, ang], -1)
        cos, sin = emb.cos(), emb.sin()
        frames = [h * w for t, h, w in grids for _ in range(t)]
        cu_full = torch.tensor([0] + list(np.cumsum(frames)), dtype=torch.int32, device=dev)
        cu_w = torch.tensor(cu_win, dtype=torch.int32, device=dev)
        max_w = max(b - a for a, b in zip(cu_win[:-1], cu_win[1:]))
        for i, blk in enumerate(self.blocks):
            if i in self.full_blocks:
                x = blk(x, cos, sin, cu_full, max(frames))
            else:
                x = blk(x, cos, sin, cu_w, max_w)
        x = self.ln_q(x).reshape(-1, self.embed * m2)
        x = self.merger_fc2(F.gelu(self.merger_fc1(x)))
        return x[torch.argsort(order)]


class Qwen2_5_VLForConditionalGeneration(Qwen2VLForConditionalGeneration):
    supports_video = False        # (its video positions follow the sampling rate: not built)

    renames = Qwen2VLForConditionalGeneration.renames

    def __init__(self, cfg: ModelConfig):
        nn.Module.__init__(self)
        from . import get_model_class

        self.cfg = cfg
        hf = cfg.hf_config
        self.image_token_id = int(hf.get("image_token_id", 151655))
        self.visual = Qwen25VisionTower(hf["vision_config"], cfg.dtype)
        self.language_model = get_model_class("Qwen2ForCausalLM")(cfg)
        tc = hf.get("text_config", hf)
        rp = tc.get("rope_parameters") or tc.get("rope_scaling") or hf.get("rope_scaling") or {}
        self.mrope_section = list(rp.get("mrope_section") or [cfg.head_dim // 2 - 2 * (cfg.head_dim // 6)] + [cfg.head_dim // 6] * 2)
        for layer in self.language_model.model.layers.values():
            layer.self_attn.mrope_section = self.mrope_section


# ------------------------------------------------------------------------------------------------------ Qwen3-VL
class Qwen3VisionTower(nn.Module):
    """Qwen3-VL vision tower: patch projection with bias, learned position embeddings on a fixed square grid that are
    bilinearly interpolated to the image's patch grid, the Qwen2-VL blocks (LayerNorm, 2-D rotary, GELU MLP), a merger,
    and DeepStack mergers that turn the hidden states after chosen blocks into extra features for the first decoder
    layers."""

    def __init__(self, vc: dict, dtype):
        super().__init__()
        self.embed, self.heads = vc["hidden_size"], vc["num_heads"]
        self.patch, self.merge, self.tpatch = vc.get("patch_size", 16), vc.get("spatial_merge_size", 2), vc.get("temporal_patch_size", 2)
        self.in_ch = vc.get("in_channels", 3)
        self.patch_dim = self.in_ch * self.tpatch * self.patch * self.patch
        self.patch_embed = ReplicatedLinear(self.patch_dim, self.embed, True, dtype)
        self.side = int(round(vc["num_position_embeddings"] ** 0.5))
        self.pos_embed = nn.Parameter(torch.zeros(vc["num_position_embeddings"], self.embed, dtype=dtype), requires_grad=False)
        self.blocks = nn.ModuleList([Qwen2VisionBlock(self.embed, self.heads, vc["intermediate_size"],
                                                      vc.get("hidden_act", "gelu_pytorch_tanh"), dtype)
                                     for _ in range(vc["depth"])])
        unit = self.embed * self.merge * self.merge
        self.deepstack_indexes = list(vc.get("deepstack_visual_indexes") or [])

        def merger(norm_dim):
            return nn.ModuleDict({"norm": LayerNorm(norm_dim, 1e-6, dtype), "fc1": ReplicatedLinear(unit, unit, True, dtype),
                                  "fc2": ReplicatedLinear(unit, vc["out_hidden_size"], True, dtype)})

        self.merger = merger(self.embed)
        self.deepstack_mergers = nn.ModuleList([merger(unit) for _ in self.deepstack_indexes])

    _angles = Qwen2VisionTower._angles

    def _pos(self, grids: list, device) -> torch.Tensor:
        """Position embeddings of every patch, in the tower's patch order (merge blocks of ``m x m`` neighbours)."""
        S, m, out = self.side, self.merge, []
        table = self.pos_embed.float()
        for t, h, w in grids:
            ys, xs = torch.linspace(0, S - 1, h, device=device), torch.linspace(0, S - 1, w, device=device)
            y0, x0 = ys.long(), xs.long()
            y1, x1 = (y0 + 1).clamp(max=S - 1), (x0 + 1).clamp(max=S - 1)
            dy, dx = (ys - y0)[:, None, None], (xs - x0)[None, :, None]
            g = lambda yy, xx: table[(yy[:, None] * S + xx[None, :])]                       # [h, w, embed]
            e = g(y0, x0) * (1 - dy) * (1 - dx) + g(y0, x1) * (1 - dy) * dx + g(y1, x0) * dy * (1 - dx) + g(y1, x1) * dy * dx
            e = e.reshape(h // m, m, w // m, m, -1).permute(0, 2, 1, 3, 4).reshape(h * w, -1)
            out.append(e.repeat(t, 1))
        return torch.cat(out)

    def _merge(self, mod, x: torch.Tensor, post_shuffle: bool) -> torch.Tensor:
        unit = self.embed * self.merge * self.merge
        x = mod["norm"](x.reshape(-1, unit)) if post_shuffle else mod["norm"](x).reshape(-1, unit)
        return mod["fc2"](F.gelu(mod["fc1"](x)))

    def forward(self, patches: torch.Tensor, grids: list):
        """``patches [N, patch_dim]`` -> ``(features [N / merge^2, hidden_text], [DeepStack features, same shape])``."""
        x = self.patch_embed(patches.to(self.patch_embed.weight.dtype))
        x = x + self._pos(grids, x.device).to(x.dtype)
        ang = self._angles(grids, x.device)
        emb = torch.cat([ang, ang], -1)
        cos, sin = emb.cos(), emb.sin()
        frames = [h * w for t, h, w in grids for _ in range(t)]
        cu = torch.tensor([0] + list(np.cumsum(frames)), dtype=torch.int32, device=x.device)
        deep = []
        for i, blk in enumerate(self.blocks):
            x = blk(x, cos, sin, cu, max(frames))
            if i in self.deepstack_indexes:
                deep.append(self._merge(self.deepstack_mergers[self.deepstack_indexes.index(i)], x, True))
        return self._merge(self.merger, x, False), deep


class Qwen3VLForConditionalGeneration(Qwen2VLForConditionalGeneration):
    """Qwen3-VL: Qwen3 decoder (per-head q / k norms) with interleaved M-RoPE, the tower above, and DeepStack - the
    features taken after chosen vision blocks are added to the hidden states of the image tokens after the first
    decoder layers.  The engine carries them beside the image features (one wider row per image token) and the
    decoder's layer loop adds level i after layer i (``attention/metadata.py:merge_multimodal_embeddings``)."""

    renames = [(r"^model\.language_model\.", "language_model.model."), (r"^model\.visual\.", "visual."),
               (r"^lm_head\.", "language_model.lm_head."), (r"^model\.(?!language_model|visual)", "language_model.model."),
               (r"^visual\.patch_embed\.proj\.", "visual.patch_embed."), (r"^visual\.pos_embed\.weight$", "visual.pos_embed"),
               (r"^visual\.blocks\.(\d+)\.attn\.", r"visual.blocks.\1."),
               (r"^visual\.blocks\.(\d+)\.mlp\.linear_fc([12])\.", r"visual.blocks.\1.fc\2."),
               (r"^visual\.merger\.linear_fc([12])\.", r"visual.merger.fc\1."),
               (r"^visual\.deepstack_merger_list\.(\d+)\.linear_fc([12])\.", r"visual.deepstack_mergers.\1.fc\2."),
               (r"^visual\.deepstack_merger_list\.(\d+)\.norm\.", r"visual.deepstack_mergers.\1.norm.")]

    def __init__(self, cfg: ModelConfig):
        nn.Module.__init__(self)
        from . import get_model_class

        self.cfg = cfg
        hf = cfg.hf_config
        self.image_token_id = int(hf.get("image_token_id", 151655))
        self.visual = Qwen3VisionTower(hf["vision_config"], cfg.dtype)
        self.language_model = get_model_class(self.decoder_arch)(cfg)
        tc = hf.get("text_config", hf)
        rp = tc.get("rope_parameters") or tc.get("rope_scaling") or hf.get("rope_scaling") or {}
        self.mrope_section = list(rp.get("mrope_section") or [24, 20, 20])
        for layer in self.language_model.model.layers.values():
            layer.self_attn.mrope_section = self.mrope_section
            layer.self_attn.mrope_interleaved = bool(rp.get("mrope_interleaved", True))
        self.language_model.model.takes_deepstack = bool(self.visual.deepstack_indexes)

    image_mean, image_std = (0.5, 0.5, 0.5), (0.5, 0.5, 0.5)          # this family's image processor
    decoder_arch = "Qwen3ForCausalLM"
    supports_video = False        # (its videos are frame groups separated by timestamp text: not built)

    @torch.no_grad()
    def encode_request(self, prompt_token_ids: list, mm: dict, device):
        orig = self.visual.forward
        deep_box = []

        def tower(patches, grids):                 # the parent's request logic with this tower's two outputs
            feats, deep = orig(patches, grids)
            deep_box.append(deep)
            return feats

        self.visual.forward = tower
        try:
            ids, (feats, pos, digest), extras = super().encode_request(prompt_token_ids, mm, device)
        finally:
            self.visual.forward = orig
        deep = deep_box[0]
        if deep:                                    # [N, hidden * (1 + levels)]: features | level 0 | level 1 | ...
            feats = torch.cat([feats] + deep, dim=-1)
        return ids, (feats, pos, digest), extras


class Qwen3VLMoeForConditionalGeneration(Qwen3VLForConditionalGeneration):
    """Qwen3-VL-MoE: the Qwen3-VL tower, M-RoPE and DeepStack over the Qwen3-MoE decoder.  Checkpoints keep the experts
    of a layer in two stacked tensors (``experts.gate_up_proj [E, 2I, H]``: gate rows then up rows;
    ``experts.down_proj [E, H, I]``); they are handed to the expert-parallel loader one expert at a time."""

    decoder_arch = "Qwen3MoeForCausalLM"

    def load_weights(self, weights: Iterable[tuple[str, torch.Tensor]]) -> set[str]:
        return super().load_weights(split_stacked_experts(weights))


def split_stacked_experts(weights):
    """``experts.gate_up_proj [E, 2I, H]`` / ``experts.down_proj [E, H, I]`` -> the per-expert tensor names the
    expert-parallel loaders take (gate rows first, then up rows)."""
    for name, w in weights:
        if name.endswith(".mlp.experts.gate_up_proj"):
            base, inter = name[: -len("gate_up_proj")], w.shape[1] // 2
            for e in range(w.shape[0]):
                yield f"{base}{e}.gate_proj.weight", w[e, :inter]
                yield f"{base}{e}.up_proj.weight", w[e, inter:]
        elif name.endswith(".mlp.experts.down_proj"):
            base = name[: -len("down_proj")]
            for e in range(w.shape[0]):
                yield f"{base}{e}.down_proj.weight", w[e]
        else:
            yield name, w


# ------------------------------------------------------------------------------------------------------ GLM-4.1V
class Glm4vVisionBlock(nn.Module):
    """RMSNorm, fused qkv (optional bias) + bias-free projection, 2-D rotary, bias-free SwiGLU MLP."""

    def __init__(self, dim: int, heads: int, inter: int, eps: float, qkv_bias: bool, dtype):
        super().__init__()
        from ..layers.basic import RMSNorm

        self.heads, self.hd = heads, dim // heads
        self.norm1, self.norm2 = RMSNorm(dim, eps, dtype), RMSNorm(dim, eps, dtype)
        self.qkv = ReplicatedLinear(dim, 3 * dim, qkv_bias, dtype)
        self.proj = ReplicatedLinear(dim, dim, False, dtype)
        self.gate_proj, self.up_proj = ReplicatedLinear(dim, inter, False, dtype), ReplicatedLinear(dim, inter, False, dtype)
        self.down_proj = ReplicatedLinear(inter, dim, False, dtype)

    def forward(self, x, cos, sin, cu, max_tokens: int):
        N, dim = x.shape
        qkv = self.qkv(self.norm1(x)).reshape(N, 3, self.heads, self.hd)
        q, k, v = qkv[:, 0], qkv[:, 1], qkv[:, 2]

        def rot(t):
            tf_ = t.float()
            a, b = tf_[..., : self.hd // 2], tf_[..., self.hd // 2:]
            return (tf_ * cos[:, None, :] + torch.cat([-b, a], -1) * sin[:, None, :]).to(t.dtype)

        a = encoder_attention(rot(q).contiguous(), rot(k).contiguous(), v.contiguous(), cu, max_tokens)
        x = x + self.proj(a.reshape(N, dim))
        y = self.norm2(x)
        return x + self.down_proj(F.silu(self.gate_proj(y)) * self.up_proj(y))


class Glm4vVisionTower(nn.Module):
    """GLM-4.1V tower: patch projection, RMSNorm, learned position embeddings sampled bicubically at every patch
    centre, RMSNorm / SwiGLU blocks with 2-D rotary, a strided convolution that merges ``m x m`` patches, and a gated
    merger MLP."""

    def __init__(self, vc: dict, dtype):
        super().__init__()
        from ..layers.basic import RMSNorm

        self.embed, self.heads = vc["hidden_size"], vc["num_heads"]
        self.patch, self.merge, self.tpatch = vc.get("patch_size", 14), vc.get("spatial_merge_size", 2), vc.get("temporal_patch_size", 2)
        self.in_ch = vc.get("in_channels", 3)
        self.patch_dim = self.in_ch * self.tpatch * self.patch * self.patch
        eps = vc.get("rms_norm_eps", 1e-5)
        out = vc["out_hidden_size"]
        self.patch_embed = ReplicatedLinear(self.patch_dim, self.embed, True, dtype)
        self.post_conv_layernorm = RMSNorm(self.embed, eps, dtype)
        self.side = vc.get("image_size", 336) // self.patch
        self.position_embedding = nn.Parameter(torch.zeros(self.side * self.side, self.embed, dtype=dtype), requires_grad=False)
        self.blocks = nn.ModuleList([Glm4vVisionBlock(self.embed, self.heads, out, eps, bool(vc.get("attention_bias", False)), dtype)
                                     for _ in range(vc["depth"])])
        self.post_layernorm = RMSNorm(self.embed, eps, dtype)
        self.downsample = ReplicatedLinear(self.embed * self.merge * self.merge, out, True, dtype)     # the strided conv
        self.merger_proj = ReplicatedLinear(out, out, False, dtype)
        self.merger_norm = LayerNorm(out, 1e-5, dtype)
        inter = vc["intermediate_size"]
        self.merger_gate, self.merger_up = ReplicatedLinear(out, inter, False, dtype), ReplicatedLinear(out, inter, False, dtype)
        self.merger_down = ReplicatedLinear(inter, out, False, dtype)

    _angles = Qwen2VisionTower._angles

    def _pos(self, grids: list, device) -> torch.Tensor:
        S, m = self.side, self.merge
        table = self.position_embedding.float().view(S, S, -1).permute(2, 0, 1)[None]            # [1, C, S, S]
        out = []
        for t, h, w in grids:
            hp = torch.arange(h, device=device)[:, None].expand(h, w).reshape(h // m, m, w // m, m).permute(0, 2, 1, 3).flatten()
            wp = torch.arange(w, device=device)[None, :].expand(h, w).reshape(h // m, m, w // m, m).permute(0, 2, 1, 3).flatten()
            gx, gy = ((wp.float() + 0.5) / w) * 2 - 1, ((hp.float() + 0.5) / h) * 2 - 1
            grid = torch.stack([gx, gy], -1)[None, :, None, :]                                     # [1, N, 1, 2]
            e = F.grid_sample(table, grid, mode="bicubic", align_corners=False, padding_mode="border")
            out.append(e[0, :, :, 0].transpose(0, 1).repeat(t, 1))
        return torch.cat(out)

    def forward(self, patches: torch.Tensor, grids: list) -> torch.Tensor:
        x = self.post_conv_layernorm(self.patch_embed(patches.to(self.patch_embed.weight.dtype)))
        ang = self._angles(grids, x.device)
        emb = torch.cat([ang, ang], -1)
        cos, sin = emb.cos(), emb.sin()
        x = x + self._pos(grids, x.device).to(x.dtype)
        frames = [h * w for t, h, w in grids for _ in range(t)]
        cu = torch.tensor([0] + list(np.cumsum(frames)), dtype=torch.int32, device=x.device)
        for blk in self.blocks:
            x = blk(x, cos, sin, cu, max(frames))
        x = self.post_layernorm(x)
        m = self.merge
        x = x.reshape(-1, m, m, self.embed).permute(0, 3, 1, 2).reshape(-1, self.embed * m * m)     # conv input order
        x = self.downsample(x)
        x = F.gelu(self.merger_norm(self.merger_proj(x)))
        return self.merger_down(F.silu(self.merger_gate(x)) * self.merger_up(x))


class Glm4vForConditionalGeneration(Qwen2VLForConditionalGeneration):
    """GLM-4.1V: the tower above over the GLM-4 decoder (extra norms after each branch, half of every head rotated in
    adjacent pairs) with M-RoPE in the chunked layout."""

    image_mean, image_std = (0.48145466, 0.4578275, 0.40821073), (0.26862954, 0.26130258, 0.27577711)
    decoder_arch = "Glm4ForCausalLM"
    supports_video = False
    renames = [(r"^model\.language_model\.", "language_model.model."), (r"^model\.visual\.", "visual."),
               (r"^lm_head\.", "language_model.lm_head."), (r"^model\.(?!language_model|visual)", "language_model.model."),
               (r"^visual\.patch_embed\.proj\.", "visual.patch_embed."),
               (r"^visual\.embeddings\.position_embedding\.weight$", "visual.position_embedding"),
               (r"^visual\.blocks\.(\d+)\.attn\.", r"visual.blocks.\1."), (r"^visual\.blocks\.(\d+)\.mlp\.", r"visual.blocks.\1."),
               (r"^visual\.merger\.proj\.", "visual.merger_proj."), (r"^visual\.merger\.post_projection_norm\.", "visual.merger_norm."),
               (r"^visual\.merger\.(gate|up|down)_proj\.", r"visual.merger_\1.")]

    def __init__(self, cfg: ModelConfig):
        nn.Module.__init__(self)
        from . import get_model_class

        self.cfg = cfg
        hf = cfg.hf_config
        self.image_token_id = int(hf.get("image_token_id", 151343))
        self.visual = Glm4vVisionTower(hf["vision_config"], cfg.dtype)
        if self.decoder_arch == "Glm4ForCausalLM":
            cfg.attention_bias = True                      # GLM-4.1V's q / k / v projections always carry a bias
        self.language_model = get_model_class(self.decoder_arch)(cfg)
        tc = hf.get("text_config", hf)
        rp = tc.get("rope_parameters") or tc.get("rope_scaling") or hf.get("rope_scaling") or {}
        self.mrope_section = list(rp.get("mrope_section") or [8, 12, 12])
        for layer in self.language_model.model.layers.values():
            layer.self_attn.mrope_section = self.mrope_section

    def load_weights(self, weights: Iterable[tuple[str, torch.Tensor]]) -> set[str]:
        def conv_as_linear():
            for name, w in weights:
                if name.endswith("visual.downsample.weight"):          # [out, C, m, m] strided convolution
                    w = w.reshape(w.shape[0], -1)
                yield name, w

        return super().load_weights(conv_as_linear())


class Glm4vMoeForConditionalGeneration(Glm4vForConditionalGeneration):
    """GLM-4.5V: the GLM-4.1V tower and M-RoPE over the GLM-4.5 mixture-of-experts decoder (NeoX-style rotation of
    half of each head; stacked expert tensors are split per expert at load)."""

    decoder_arch = "Glm4MoeForCausalLM"

    def load_weights(self, weights: Iterable[tuple[str, torch.Tensor]]) -> set[str]:
        return super().load_weights(split_stacked_experts(weights))
