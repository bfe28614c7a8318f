"""InternVL (Hugging Face format): InternViT tower -> pixel-shuffle (2x2 patches folded into channels) -> LayerNorm +
2-layer projector -> a text decoder of this package (Qwen2 / InternLM2 / Llama).

    tower layer:   x += lambda_1 * attn(LN(x));   x += lambda_2 * mlp(LN(x))        (layer scale, GELU MLP)

The engine-facing half - placeholder expansion, feature merge per prefill chunk, image-salted prefix cache - is the
LLaVA class's (``models/llava.py``); this file only swaps the encoder.
Parity: InternVLForConditionalGeneration / InternVLChatModel rows of the reference's multimodal table
(docs/models/supported_models.md:80-81).
"""
from __future__ import annotations

import re
from typing import Iterable

import torch
import torch.nn as nn
import torch.nn.functional as F

from .. import _custom_ops as ops
from ..config import ModelConfig
from ..layers.basic import LayerNorm, RMSNorm
from ..layers.linear import ReplicatedLinear
from ..layers.mm_encoder_attention import encoder_attention
from .llava import _ACT, LlavaForConditionalGeneration


def _pair(v):
    return (v, v) if isinstance(v, int) else tuple(v)


class InternVitLayer(nn.Module):
    def __init__(self, vc: dict, dtype):
        super().__init__()
        hid, heads = vc["hidden_size"], vc["num_attention_heads"]
        self.heads, self.hd = heads, hid // heads
        eps = vc.get("layer_norm_eps", 1e-6)
        norm = (lambda: RMSNorm(hid, eps, dtype)) if vc.get("norm_type", "layer_norm") == "rms_norm" else (lambda: LayerNorm(hid, eps, dtype))
        assert not vc.get("use_qk_norm", False), "InternViT q/k norm is not supported"
        self.layernorm_before, self.layernorm_after = norm(), norm()
        self.qkv_proj = ReplicatedLinear(hid, 3 * hid, bool(vc.get("attention_bias", False)), dtype)
        self.projection_layer = ReplicatedLinear(hid, hid, True, dtype)
        self.fc1 = ReplicatedLinear(hid, vc["intermediate_size"], True, dtype)
        self.fc2 = ReplicatedLinear(vc["intermediate_size"], hid, True, dtype)
        self.lambda_1 = nn.Parameter(torch.ones(hid, dtype=dtype), requires_grad=False)
        self.lambda_2 = nn.Parameter(torch.ones(hid, dtype=dtype), requires_grad=False)
        self.act = _ACT.get(vc.get("hidden_act", "gelu"), "gelu")

    def forward(self, x, cu, tokens):
        T, hid = x.shape
        qkv = self.qkv_proj(self.layernorm_before(x)).reshape(T, 3, self.heads, self.hd)
        a = encoder_attention(qkv[:, 0], qkv[:, 1], qkv[:, 2], cu, tokens)
        x = x + self.lambda_1 * self.projection_layer(a.reshape(T, hid))
        return x + self.lambda_2 * self.fc2(ops.activation(self.fc1(self.layernorm_after(x)), self.act))


class InternVitTower(nn.Module):
    def __init__(self, vc: dict, dtype, num_layers: int):
        super().__init__()
        hid = vc["hidden_size"]
        (self.size, _), (self.patch, _) = _pair(vc["image_size"]), _pair(vc["patch_size"])
        self.grid = self.size // self.patch
        self.tokens = self.grid * self.grid + 1
        self.cls_token = nn.Parameter(torch.zeros(1, 1, hid, dtype=dtype), requires_grad=False)
        self.position_embeddings = nn.Parameter(torch.zeros(1, self.tokens, hid, dtype=dtype), requires_grad=False)
        self.patch_weight = nn.Parameter(torch.zeros(hid, 3 * self.patch * self.patch, dtype=dtype), requires_grad=False)
        self.patch_bias = nn.Parameter(torch.zeros(hid, dtype=dtype), requires_grad=False)
        self.layers = nn.ModuleList([InternVitLayer(vc, dtype) for _ in range(num_layers)])

    def forward(self, pixels: torch.Tensor) -> torch.Tensor:
        n, p, g = pixels.shape[0], self.patch, self.grid
        x = pixels.to(self.patch_weight.dtype).reshape(n, 3, g, p, g, p).permute(0, 2, 4, 1, 3, 5).reshape(n * g * g, 3 * p * p)
        x = F.linear(x, self.patch_weight, self.patch_bias).reshape(n, g * g, -1)
        x = (torch.cat([self.cls_token.expand(n, 1, -1), x], 1) + self.position_embeddings).reshape(n * self.tokens, -1)
        cu = torch.arange(0, (n + 1) * self.tokens, self.tokens, dtype=torch.int32, device=x.device)
        for layer in self.layers:
            x = layer(x, cu, self.tokens)
        return x.reshape(n, self.tokens, -1)


class InternVLForConditionalGeneration(LlavaForConditionalGeneration):
    renames = [(r"^model\.language_model\.(?!model\.|lm_head\.)", "language_model.model."),
               (r"^model\.language_model\.model\.", "language_model.model."), (r"^lm_head\.", "language_model.lm_head."),
               (r"^model\.vision_tower\.", "vision_tower."), (r"^model\.multi_modal_projector\.", "multi_modal_projector."),
               (r"^vision_tower\.embeddings\.patch_embeddings\.projection\.weight$", "vision_tower.patch_weight"),
               (r"^vision_tower\.embeddings\.patch_embeddings\.projection\.bias$", "vision_tower.patch_bias"),
               (r"^vision_tower\.embeddings\.", "vision_tower."), (r"^vision_tower\.encoder\.layer\.", "vision_tower.layers."),
               (r"\.attention\.projection_layer\.", ".projection_layer."), (r"\.mlp\.fc([12])\.", r".fc\1.")]
    qkv_pattern = r"(vision_tower\.layers\.\d+)\.attention\.([qkv])_proj\.(weight|bias)$"

    def __init__(self, cfg: ModelConfig):
        nn.Module.__init__(self)
        from . import get_model_class

        self.cfg = cfg
        hf = cfg.hf_config
        vc = hf["vision_config"]
        self.image_token_id = int(hf.get("image_token_id", hf.get("image_token_index", 151667)))
        layer = hf.get("vision_feature_layer", -1)
        total = vc["num_hidden_layers"]
        keep = total if layer == -1 else (total + layer + 1 if layer < 0 else layer)
        self.select = hf.get("vision_feature_select_strategy", "default")
        self.ratio = float(hf.get("downsample_ratio", 0.5))
        self.vision_tower = InternVitTower(vc, cfg.dtype, keep)
        fold = int(round(1 / self.ratio)) ** 2
        vh = vc["hidden_size"] * fold
        self.multi_modal_projector = nn.ModuleDict({
            "layer_norm": LayerNorm(vh, 1e-5, cfg.dtype),
            "linear_1": ReplicatedLinear(vh, cfg.hidden_size, True, cfg.dtype),
            "linear_2": ReplicatedLinear(cfg.hidden_size, cfg.hidden_size, True, cfg.dtype)})
        self.proj_act = _ACT.get(hf.get("projector_hidden_act", "gelu"), "gelu")
        text_arch = (hf.get("text_config", {}).get("architectures") or ["Qwen2ForCausalLM"])[0]
        if text_arch not in ("Qwen2ForCausalLM", "LlamaForCausalLM", "InternLM2ForCausalLM", "Qwen3ForCausalLM"):
            text_arch = {"qwen2": "Qwen2ForCausalLM", "llama": "LlamaForCausalLM", "qwen3": "Qwen3ForCausalLM"}.get(
                hf.get("text_config", {}).get("model_type", "qwen2"), "Qwen2ForCausalLM")
        self.language_model = get_model_class(text_arch)(cfg)
        g = int(self.vision_tower.grid * self.ratio)
        self.tokens_per_image = g * g

    @torch.no_grad()
    def embed_multimodal(self, pixel_values: torch.Tensor) -> torch.Tensor:
        feats = self.vision_tower(pixel_values)
        if self.select == "default":
            feats = feats[:, 1:]
        n, t, c = feats.shape
        g, r = int(t ** 0.5), self.ratio
        x = feats.reshape(n, g, g, c)
        x = x.reshape(n, g, int(g * r), int(c / r)).permute(0, 2, 1, 3).contiguous()        # fold 2 columns into channels
        x = x.reshape(n, int(g * r), int(g * r), int(c / (r * r))).permute(0, 2, 1, 3).contiguous()   # then 2 rows
        x = x.reshape(n * self.tokens_per_image, -1)
        x = self.multi_modal_projector["layer_norm"](x)
        x = self.multi_modal_projector["linear_2"](ops.activation(self.multi_modal_projector["linear_1"](x), self.proj_act))
        return x.reshape(n, self.tokens_per_image, -1)

    def preprocess(self, image) -> torch.Tensor:
        S = self.vision_tower.size
        if not isinstance(image, torch.Tensor):
            import numpy as np

            image = torch.from_numpy(np.asarray(image.convert("RGB"))).permute(2, 0, 1)
        x = image.float() / (255.0 if image.dtype == torch.uint8 else 1.0)
        x = F.interpolate(x[None], size=(S, S), mode="bicubic", align_corners=False)[0].clamp(0, 1)
        mean = torch.tensor([0.485, 0.456, 0.406]).view(3, 1, 1)
        std = torch.tensor([0.229, 0.224, 0.225]).view(3, 1, 1)
        return (x - mean) / std


class InternVLChatModel(InternVLForConditionalGeneration):
    """The original InternVL export (``vision_model.*`` with fused ``attn.qkv``, ``ls1`` / ``ls2``, ``mlp1.{0,1,3}``,
    ``llm_config``): the same graph under other names.  The image-context token is a tokenizer entry there, so its id
    comes from ``img_context_token_id`` in the config when present (default: ``<IMG_CONTEXT>`` of the Qwen2 tokenizer)."""
    renames = [(r"^language_model\.lm_head\.", "language_model.lm_head."),
               (r"^vision_model\.embeddings\.class_embedding$", "vision_tower.cls_token"),
               (r"^vision_model\.embeddings\.position_embedding$", "vision_tower.position_embeddings"),
               (r"^vision_model\.embeddings\.patch_embedding\.weight$", "vision_tower.patch_weight"),
               (r"^vision_model\.embeddings\.patch_embedding\.bias$", "vision_tower.patch_bias"),
               (r"^vision_model\.encoder\.layers\.", "vision_tower.layers."),
               (r"\.attn\.qkv\.", ".qkv_proj."), (r"\.attn\.proj\.", ".projection_layer."),
               (r"\.ls1$", ".lambda_1"), (r"\.ls2$", ".lambda_2"),
               (r"\.norm1\.", ".layernorm_before."), (r"\.norm2\.", ".layernorm_after."), (r"\.mlp\.fc([12])\.", r".fc\1."),
               (r"^mlp1\.0\.", "multi_modal_projector.layer_norm."), (r"^mlp1\.1\.", "multi_modal_projector.linear_1."),
               (r"^mlp1\.3\.", "multi_modal_projector.linear_2.")]

    def __init__(self, cfg: ModelConfig):
        hf = cfg.hf_config
        vc = dict(hf["vision_config"])
        vc.setdefault("attention_bias", bool(vc.get("qkv_bias", True)))
        vc.setdefault("use_qk_norm", bool(vc.get("qk_normalization", False)))
        hf = dict(hf, vision_config=vc, vision_feature_layer=hf.get("select_layer", -1),
                  image_token_id=hf.get("img_context_token_id", hf.get("image_token_id", 151667)))
        hf.setdefault("text_config", hf.get("llm_config", {}))
        cfg.hf_config = hf
        super().__init__(cfg)
