"""LLaVA-1.5 style vision-language models: CLIP vision transformer -> 2-layer projector -> a text decoder of this package.

    pixel_values [n, 3, S, S] -> patches -> [CLS | patch tokens] + positions -> pre-LN
        -> encoder layers (LN, bidirectional attention over each image's tokens, LN, quick-GELU MLP)
        -> hidden state of layer ``vision_feature_layer`` without CLS -> linear, GELU, linear -> [n, tokens, hidden_text]

The projected rows replace the rows of the prompt's image-placeholder tokens in the decoder's input embeddings
(``attention/metadata.py:merge_multimodal_embeddings`` inside the decoder's embedding step); everything after that is
the ordinary text path - paged KV, chunked prefill, CUDA-graph decode.  The vision attention runs on the non-causal path
of the varlen tcgen05 kernel (``layers/mm_encoder_attention.py``).

Parity: LlavaForConditionalGeneration in the reference's multimodal table (docs/models/supported_models.md:82) and its
``MMEncoderAttention`` layer (registry/custom_ops/layers/attention/mm_encoder_attention.py:17-122).
"""
from __future__ import annotations

import re
from typing import Iterable

import torch
import torch.nn as nn
import torch.nn.functional as F

from .. import _custom_ops as ops
from ..config import ModelConfig
from ..layers.basic import LayerNorm
from ..layers.linear import ReplicatedLinear
from ..layers.mm_encoder_attention import encoder_attention

_ACT = {"quick_gelu": "gelu_quick", "gelu": "gelu", "gelu_pytorch_tanh": "gelu_tanh", "gelu_new": "gelu_new"}


class ClipEncoderLayer(nn.Module):
    def __init__(self, hid: int, inter: int, heads: int, eps: float, act: str, dtype):
        super().__init__()
        self.heads, self.hd = heads, hid // heads
        self.layer_norm1 = LayerNorm(hid, eps, dtype)
        self.layer_norm2 = LayerNorm(hid, eps, dtype)
        self.qkv_proj = ReplicatedLinear(hid, 3 * hid, True, dtype)
        self.out_proj = ReplicatedLinear(hid, hid, True, dtype)
        self.fc1 = ReplicatedLinear(hid, inter, True, dtype)
        self.fc2 = ReplicatedLinear(inter, hid, True, dtype)
        self.act = _ACT.get(act, act)

    def forward(self, x: torch.Tensor, cu: torch.Tensor, tokens: int) -> torch.Tensor:
        T, hid = x.shape
        qkv = self.qkv_proj(self.layer_norm1(x)).reshape(T, 3, self.heads, self.hd)
        a = encoder_attention(qkv[:, 0], qkv[:, 1], qkv[:, 2], cu, tokens)
        x = x + self.out_proj(a.reshape(T, hid))
        return x + self.fc2(ops.activation(self.fc1(self.layer_norm2(x)), self.act))


class ClipVisionTower(nn.Module):
    def __init__(self, vc: dict, dtype, num_layers: int):
        super().__init__()
        hid, self.patch, self.size = vc["hidden_size"], vc["patch_size"], vc["image_size"]
        self.grid = self.size // self.patch
        self.tokens = self.grid * self.grid + 1
        eps = vc.get("layer_norm_eps", 1e-5)
        self.class_embedding = nn.Parameter(torch.zeros(hid, dtype=dtype), requires_grad=False)
        self.patch_embedding = nn.Parameter(torch.zeros(hid, 3 * self.patch * self.patch, dtype=dtype), requires_grad=False)
        self.position_embedding = nn.Parameter(torch.zeros(self.tokens, hid, dtype=dtype), requires_grad=False)
        self.pre_layrnorm = LayerNorm(hid, eps, dtype)
        self.layers = nn.ModuleList([ClipEncoderLayer(hid, vc["intermediate_size"], vc["num_attention_heads"], eps,
                                                      vc.get("hidden_act", "quick_gelu"), dtype) for _ in range(num_layers)])

    def forward(self, pixels: torch.Tensor) -> torch.Tensor:
        """``pixels [n, 3, S, S]`` -> ``[n, tokens, hidden]`` after the last kept layer."""
        n, p, g = pixels.shape[0], self.patch, self.grid
        dt = self.patch_embedding.dtype
        x = pixels.to(dt).reshape(n, 3, g, p, g, p).permute(0, 2, 4, 1, 3, 5).reshape(n * g * g, 3 * p * p)
        x = F.linear(x, self.patch_embedding).reshape(n, g * g, -1)
        x = torch.cat([self.class_embedding.expand(n, 1, -1), x], 1) + self.position_embedding
        x = self.pre_layrnorm(x.reshape(n * self.tokens, -1))
        cu = torch.arange(0, (n + 1) * self.tokens, self.tokens, dtype=torch.int32, device=x.device)
        for layer in self.layers:
            x = layer(x, cu, self.tokens)
        return x.reshape(n, self.tokens, -1)


class LlavaForConditionalGeneration(nn.Module):
    is_multimodal = True
    qkv_pattern = r"(vision_tower\.layers\.\d+)\.self_attn\.([qkv])_proj\.(weight|bias)$"
    renames = [(r"^model\.language_model\.model\.", "language_model.model."),
               (r"^model\.language_model\.(?!model\.|lm_head\.)", "language_model.model."),
               (r"^lm_head\.", "language_model.lm_head."),
               (r"^model\.vision_tower\.", "vision_tower."), (r"^model\.multi_modal_projector\.", "multi_modal_projector."),
               (r"^vision_tower\.vision_model\.embeddings\.patch_embedding\.weight$", "vision_tower.patch_embedding"),
               (r"^vision_tower\.vision_model\.embeddings\.class_embedding$", "vision_tower.class_embedding"),
               (r"^vision_tower\.vision_model\.embeddings\.position_embedding\.weight$", "vision_tower.position_embedding"),
               (r"^vision_tower\.vision_model\.encoder\.layers\.", "vision_tower.layers."),
               (r"^vision_tower\.vision_model\.pre_layrnorm\.", "vision_tower.pre_layrnorm."),
               (r"\.self_attn\.out_proj\.", ".out_proj."), (r"\.mlp\.fc([12])\.", r".fc\1.")]

    def __init__(self, cfg: ModelConfig):
        super().__init__()
        from . import get_model_class

        self.cfg = cfg
        hf = cfg.hf_config
        vc = hf["vision_config"]
        self.image_token_id = int(hf.get("image_token_index", hf.get("image_token_id", 32000)))
        layer = hf.get("vision_feature_layer", -2)
        assert isinstance(layer, int), "one vision feature layer is supported"
        total = vc["num_hidden_layers"]
        keep = total + layer + 1 if layer < 0 else layer          # hidden_states[layer]: output of `keep` layers
        self.select = hf.get("vision_feature_select_strategy", "default")
        self.vision_tower = ClipVisionTower(vc, cfg.dtype, keep)
        bias = bool(hf.get("multimodal_projector_bias", True))
        self.multi_modal_projector = nn.ModuleDict({
            "linear_1": ReplicatedLinear(vc["hidden_size"], cfg.hidden_size, bias, cfg.dtype),
            "linear_2": ReplicatedLinear(cfg.hidden_size, cfg.hidden_size, bias, cfg.dtype)})
        self.proj_act = _ACT.get(hf.get("projector_hidden_act", "gelu"), "gelu")
        text_arch = (hf.get("text_config", {}).get("architectures") or ["LlamaForCausalLM"])[0]
        self.language_model = get_model_class(text_arch)(cfg)
        self.tokens_per_image = self.vision_tower.tokens - (1 if self.select == "default" else 0)

    # ---- multimodal interface (engine/multimodal.py) ---------------------------------
    @torch.no_grad()
    def embed_multimodal(self, pixel_values: torch.Tensor) -> torch.Tensor:
        """``[n, 3, S, S]`` -> ``[n, tokens_per_image, hidden_text]``."""
        feats = self.vision_tower(pixel_values)
        if self.select == "default":
            feats = feats[:, 1:]
        n, t, hv = feats.shape
        x = self.multi_modal_projector["linear_1"](feats.reshape(n * t, hv))
        x = self.multi_modal_projector["linear_2"](ops.activation(x, self.proj_act))
        return x.reshape(n, t, -1)

    def preprocess(self, image) -> torch.Tensor:
        """A PIL image / ``[3, H, W]`` uint8 or float tensor -> CLIP-normalised ``[3, S, S]``."""
        S = self.vision_tower.size
        if not isinstance(image, torch.Tensor):
            import numpy as np

            image = torch.from_numpy(np.asarray(image.convert("RGB"))).permute(2, 0, 1)
        x = image.float() / (255.0 if image.dtype == torch.uint8 else 1.0)
        x = F.interpolate(x[None], size=(S, S), mode="bicubic", align_corners=False)[0].clamp(0, 1)
        mean = torch.tensor([0.48145466, 0.4578275, 0.40821073]).view(3, 1, 1)
        std = torch.tensor([0.26862954, 0.26130258, 0.27577711]).view(3, 1, 1)
        return (x - mean) / std

    # ---- engine interface: the text decoder's -------------------------------------------
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

    # ---- weights -----------------------------------------------------------------------------
    def load_weights(self, weights: Iterable[tuple[str, torch.Tensor]]) -> set[str]:
        params = dict(self.named_parameters())
        text, loaded, qkv = [], set(), {}
        for name, w in weights:
            for pat, rep in self.renames:
                name = re.sub(pat, rep, name)
            if name.startswith("language_model."):
                text.append((name[len("language_model."):], w))
                continue
            m = re.match(self.qkv_pattern, name)
            if m:                                   # q, k, v of a vision layer are fused into one GEMM
                if int(m.group(1).rsplit(".", 1)[1]) < len(self.vision_tower.layers):
                    qkv.setdefault((m.group(1), m.group(3)), {})[m.group(2)] = w
                continue
            if name in ("vision_tower.patch_embedding", "vision_tower.patch_weight"):
                w = w.reshape(w.shape[0], -1)
            if name in params:
                params[name].data.copy_(w.reshape(params[name].shape))
                loaded.add(name)
        for (layer, kind), parts in qkv.items():
            target = f"{layer}.qkv_proj.{kind}"
            params[target].data.copy_(torch.cat([parts["q"], parts["k"], parts["v"]], 0))
            loaded.add(target)
        got = self.language_model.load_weights(text)
        lm = self.language_model
        if "lm_head.weight" not in got and getattr(lm, "lm_head", None) is not None and lm.lm_head is not lm.model.embed_tokens:
            # wrappers that tie the head at the top level save no lm_head tensor whatever the decoder's own flag says
            lm.lm_head.weight.data.copy_(lm.model.embed_tokens.weight.data)
        loaded |= {f"language_model.{n}" for n in got}
        return loaded


# ------------------------------------------------------------------------------------------ LLaVA-NeXT (any resolution)
def select_best_resolution(original_hw: tuple, candidates: list) -> tuple:
    """The candidate ``(height, width)`` that keeps most of the image's pixels after an aspect-preserving resize, and
    among equals wastes the least canvas (the rule LLaVA-NeXT's processor and model both apply)."""
    oh, ow = original_hw
    best, best_eff, best_waste = None, 0, float("inf")
    for h, w in candidates:
        scale = min(w / ow, h / oh)
        eff = min(int(ow * scale) * int(oh * scale), ow * oh)
        waste = w * h - eff
        if eff > best_eff or (eff == best_eff and waste < best_waste):
            best, best_eff, best_waste = (h, w), eff, waste
    return best


def unpad_features(x: torch.Tensor, original_hw: tuple) -> torch.Tensor:
    """``x [C, H, W]`` is the feature map of an image that was resized with its aspect ratio kept and padded to the
    canvas: cut the rows (or columns) that only saw padding."""
    oh, ow = original_hw
    H, W = x.shape[1:]
    if ow / oh > W / H:
        new_h = int(round(oh * (W / ow), 7))
        pad = (H - new_h) // 2
        return x[:, pad: H - pad, :]
    new_w = int(round(ow * (H / oh), 7))
    pad = (W - new_w) // 2
    return x[:, :, pad: W - pad]


class LlavaNextForConditionalGeneration(LlavaForConditionalGeneration):
    """LLaVA-NeXT (1.6): the image is shown to the CLIP tower once whole (resized to the tower's square) and once as
    a grid of tower-sized tiles cut from the best-fitting canvas of ``image_grid_pinpoints``; the tile features are
    laid out as one feature map, the padding rows / columns are cut, a learned ``image_newline`` vector ends every
    row, and base + grid features replace the prompt's placeholder run.  The number of image tokens therefore depends
    on the image size."""

    renames = LlavaForConditionalGeneration.renames + [(r"^model\.image_newline$", "image_newline")]

    def __init__(self, cfg: ModelConfig):
        super().__init__(cfg)
        hf = cfg.hf_config
        self.pinpoints = [tuple(p) for p in hf.get("image_grid_pinpoints",
                                                   [[336, 672], [672, 336], [672, 672], [1008, 336], [336, 1008]])]
        self.image_newline = nn.Parameter(torch.zeros(cfg.hidden_size, dtype=cfg.dtype), requires_grad=False)

    # ---- preprocessing: one image -> [1 + tiles, 3, S, S] and its original (h, w) --------------------------------
    def tiles_of(self, image) -> tuple:
        S = self.vision_tower.size
        if not isinstance(image, torch.Tensor):
            import numpy as np

            image = torch.from_numpy(np.asarray(image.convert("RGB"))).permute(2, 0, 1)
        x = image.float() / (255.0 if image.dtype == torch.uint8 else 1.0)
        oh, ow = x.shape[1:]
        ch, cw = select_best_resolution((oh, ow), self.pinpoints)
        import math

        if cw / ow < ch / oh:                     # the width binds: fill it, round the height up
            nw, nh = cw, min(math.ceil(oh * (cw / ow)), ch)
        else:
            nh, nw = ch, min(math.ceil(ow * (ch / oh)), cw)
        resized = F.interpolate(x[None], size=(nh, nw), mode="bicubic", align_corners=False)[0].clamp(0, 1)
        canvas = torch.zeros(3, ch, cw)
        top, left = (ch - nh) // 2, (cw - nw) // 2
        canvas[:, top: top + nh, left: left + nw] = resized
        tiles = canvas.unfold(1, S, S).unfold(2, S, S).permute(1, 2, 0, 3, 4).reshape(-1, 3, S, S)   # row-major grid
        base = F.interpolate(x[None], size=(S, S), mode="bicubic", align_corners=False)[0].clamp(0, 1)
        mean = torch.tensor(getattr(self, "image_mean", (0.48145466, 0.4578275, 0.40821073))).view(1, 3, 1, 1)
        std = torch.tensor(getattr(self, "image_std", (0.26862954, 0.26130258, 0.27577711))).view(1, 3, 1, 1)
        return (torch.cat([base[None], tiles]) - mean) / std, (oh, ow)

    # ---- features of one image: [tokens, hidden] ------------------------------------------------------------------
    def pack_features(self, feats: torch.Tensor, original_hw: tuple) -> torch.Tensor:
        """``feats [1 + tiles, per, hidden]`` (projected tower outputs of the whole image and of the tiles)."""
        S, side = self.vision_tower.size, int(round(feats.shape[1] ** 0.5))
        newline = self.image_newline.to(feats.dtype)
        if feats.shape[0] == 1:
            return torch.cat([feats[0], newline[None]])
        ch, cw = select_best_resolution(original_hw, self.pinpoints)
        gh, gw = ch // S, cw // S
        grid = feats[1:].reshape(gh, gw, side, side, -1).permute(4, 0, 2, 1, 3).reshape(-1, gh * side, gw * side)
        grid = unpad_features(grid, original_hw)
        grid = torch.cat([grid, newline[:, None, None].expand(-1, grid.shape[1], 1)], dim=-1)
        return torch.cat([feats[0], grid.flatten(1).transpose(0, 1)])

    @torch.no_grad()
    def encode_request(self, prompt_token_ids: list, mm: dict, device):
        """``mm``: ``{"image": image | [images]}`` (PIL / ``[3, H, W]`` tensors), or the processor's outputs
        ``{"pixel_values": [n, 1 + tiles, 3, S, S] (zero-padded tiles allowed), "image_sizes": [n, 2]}``.  The prompt
        holds one placeholder per image or the already expanded runs."""
        import hashlib

        import numpy as np

        if "pixel_values" in mm:
            sizes = [tuple(int(v) for v in s) for s in torch.as_tensor(mm["image_sizes"]).tolist()]
            S = self.vision_tower.size
            stacks = []
            for pv, hw in zip(mm["pixel_values"], sizes):
                ch, cw = select_best_resolution(hw, self.pinpoints)
                stacks.append(pv[: 1 + (ch // S) * (cw // S)])           # drop the batch padding tiles
        else:
            imgs = mm["image"] if isinstance(mm["image"], (list, tuple)) else [mm["image"]]
            stacks, sizes = zip(*[self.tiles_of(im) for im in imgs])
        per_image = []
        for st, hw in zip(stacks, sizes):
            f = self.embed_multimodal(st.to(device=device, dtype=self.image_newline.dtype))
            per_image.append(self.pack_features(f, hw))
        tok = self.image_token_id
        runs, ids = [], []
        count = sum(1 for t in prompt_token_ids if t == tok)
        if count == len(per_image):                                      # one placeholder per image: expand
            k = 0
            for t in prompt_token_ids:
                if t == tok:
                    ids.extend([tok] * per_image[k].shape[0])
                    k += 1
                else:
                    ids.append(t)
        elif count == sum(f.shape[0] for f in per_image):
            ids = list(prompt_token_ids)
        else:
            raise ValueError(f"prompt has {count} image placeholder tokens; the images need "
                             f"{[int(f.shape[0]) for f in per_image]}")
        pos = np.asarray([i for i, t in enumerate(ids) if t == tok], dtype=np.int64)
        h = hashlib.sha256()
        for st in stacks:
            h.update(st.detach().float().cpu().numpy().tobytes())
        return ids, (torch.cat(per_image), pos, h.hexdigest()[:16]), None


# ------------------------------------------------------------------------------------------ LLaVA-OneVision (SigLIP tower)
class SiglipVisionTower(nn.Module):
    """SigLIP vision encoder as the LLaVA-OneVision family uses it: patch projection with bias, learned position
    embeddings, no class token and no norm before the encoder; the features are the output of the last kept layer."""

    def __init__(self, vc: dict, dtype, num_layers: int):
        super().__init__()
        hid, self.patch, self.size = vc["hidden_size"], vc["patch_size"], vc["image_size"]
        self.grid = self.size // self.patch
        self.tokens = self.grid * self.grid
        eps = vc.get("layer_norm_eps", 1e-6)
        self.patch_embedding = nn.Parameter(torch.zeros(hid, 3 * self.patch * self.patch, dtype=dtype), requires_grad=False)
        self.patch_bias = nn.Parameter(torch.zeros(hid, dtype=dtype), requires_grad=False)
        self.position_embedding = nn.Parameter(torch.zeros(self.tokens, hid, dtype=dtype), requires_grad=False)
        self.layers = nn.ModuleList([ClipEncoderLayer(hid, vc["intermediate_size"], vc["num_attention_heads"], eps,
                                                      vc.get("hidden_act", "gelu_pytorch_tanh"), dtype) for _ in range(num_layers)])

    def forward(self, pixels: torch.Tensor) -> torch.Tensor:
        n, p, g = pixels.shape[0], self.patch, self.grid
        dt = self.patch_embedding.dtype
        x = pixels.to(dt).reshape(n, 3, g, p, g, p).permute(0, 2, 4, 1, 3, 5).reshape(n * g * g, 3 * p * p)
        x = (F.linear(x, self.patch_embedding, self.patch_bias).reshape(n, g * g, -1) + self.position_embedding).reshape(n * self.tokens, -1)
        cu = torch.arange(0, (n + 1) * self.tokens, self.tokens, dtype=torch.int32, device=x.device)
        for layer in self.layers:
            x = layer(x, cu, self.tokens)
        return x.reshape(n, self.tokens, -1)


class LlavaOnevisionForConditionalGeneration(LlavaNextForConditionalGeneration):
    """LLaVA-OneVision: the any-resolution packing of LLaVA-NeXT over a SigLIP tower (all of its tokens are image
    tokens), with one more step - a feature map that would exceed ``anyres_max_N`` tower images' worth of tokens is
    shrunk bilinearly before the newline column is added."""

    renames = LlavaNextForConditionalGeneration.renames + [
        (r"^vision_tower\.vision_model\.embeddings\.patch_embedding\.bias$", "vision_tower.patch_bias"),
        (r"^vision_tower\.vision_model\.post_layernorm\..*$", "vision_tower.unused_post_layernorm"),
        (r"^vision_tower\.vision_model\.head\..*$", "vision_tower.unused_head")]

    def __init__(self, cfg: ModelConfig):
        super().__init__(cfg)
        hf = cfg.hf_config
        vc = hf["vision_config"]
        layer = hf.get("vision_feature_layer", -1)
        total = vc["num_hidden_layers"]
        keep = total + layer + 1 if layer < 0 else layer
        self.select = hf.get("vision_feature_select_strategy", "full")
        self.vision_tower = SiglipVisionTower(vc, cfg.dtype, keep)
        self.tokens_per_image = self.vision_tower.tokens
        self.max_tiles = int(str(hf.get("vision_aspect_ratio", "anyres_max_9")).replace("anyres_max_", ""))
        self.image_mean, self.image_std = (0.5, 0.5, 0.5), (0.5, 0.5, 0.5)

    @torch.no_grad()
    def embed_multimodal(self, pixel_values: torch.Tensor) -> torch.Tensor:
        feats = self.vision_tower(pixel_values)                          # every token is an image token (no class token)
        n, t, hv = feats.shape
        x = self.multi_modal_projector["linear_1"](feats.reshape(n * t, hv))
        x = self.multi_modal_projector["linear_2"](ops.activation(x, self.proj_act))
        return x.reshape(n, t, -1)

    def pack_features(self, feats: torch.Tensor, original_hw: tuple) -> torch.Tensor:
        import math

        S, side = self.vision_tower.size, int(round(feats.shape[1] ** 0.5))
        newline = self.image_newline.to(feats.dtype)
        if feats.shape[0] == 1:
            return torch.cat([feats[0], newline[None]])
        ch, cw = select_best_resolution(original_hw, self.pinpoints)
        gh, gw = ch // S, cw // S
        grid = feats[1:].reshape(gh, gw, side, side, -1).permute(4, 0, 2, 1, 3).reshape(-1, gh * side, gw * side)
        grid = unpad_features(grid, original_hw)
        _, H, W = grid.shape
        ratio = math.sqrt(H * W / (self.max_tiles * side * side))
        if ratio > 1.1:
            grid = F.interpolate(grid[None].float(), [int(H // ratio), int(W // ratio)], mode="bilinear")[0].to(feats.dtype)
        grid = torch.cat([grid, newline[:, None, None].expand(-1, grid.shape[1], 1)], dim=-1)
        return torch.cat([feats[0], grid.flatten(1).transpose(0, 1)])
