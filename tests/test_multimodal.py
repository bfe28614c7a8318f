"""Vision-language path: CLIP tower + projector + text decoder against Hugging Face's LLaVA (tiny random checkpoint,
fp32, CPU), image features merged at the placeholder rows across chunked prefill, prefix-cache keys salted by image."""
import pytest
import torch

tf = pytest.importorskip("transformers")

IMG_TOK = 500


def _hf_llava(tmp_path):
    torch.manual_seed(0)
    vc = tf.CLIPVisionConfig(hidden_size=64, intermediate_size=128, num_hidden_layers=3, num_attention_heads=4,
                             image_size=28, patch_size=14, projection_dim=32)
    tc = tf.LlamaConfig(vocab_size=512, hidden_size=128, intermediate_size=256, num_hidden_layers=2, num_attention_heads=4,
                        num_key_value_heads=2, max_position_embeddings=256)
    c = tf.LlavaConfig(vision_config=vc, text_config=tc, image_token_index=IMG_TOK, vision_feature_layer=-2,
                       vision_feature_select_strategy="default", image_seq_length=4)
    hf = tf.LlavaForConditionalGeneration(c).eval().float()
    with torch.no_grad():
        for p in hf.parameters():
            if p.dim() == 1:
                p.add_(0.1 * torch.randn_like(p))
            else:
                p.mul_(3.0)
    hf.save_pretrained(str(tmp_path))
    return hf


def _want(hf, ids, pixels, n=6):
    with torch.no_grad():
        out = hf.generate(input_ids=torch.tensor([ids]), pixel_values=pixels, max_new_tokens=n, do_sample=False,
                          eos_token_id=None, pad_token_id=0)
    return out[0, len(ids):].tolist()


@pytest.mark.parametrize("chunk", [64, 5])
def test_llava_matches_hugging_face(tmp_path, chunk):
    from vllm_metax_b200 import LLM, SamplingParams

    hf = _hf_llava(tmp_path)
    llm = LLM(str(tmp_path), dtype="float32", device="cpu", max_model_len=128, num_gpu_blocks=32, block_size=16,
              max_num_batched_tokens=chunk, enable_prefix_caching=True)
    g = torch.Generator().manual_seed(1)
    img_a, img_b = torch.randn(1, 3, 28, 28, generator=g), torch.randn(1, 3, 28, 28, generator=g)
    two = torch.cat([img_a, img_b])
    expanded = [5, 9] + [IMG_TOK] * 4 + [33, 100, 7, 8, 200, 31, 2, 17, 45, 301, 77, 12]          # 4 tokens per image
    short = [5, 9, IMG_TOK, 33, 100, 7, 8, 200, 31, 2, 17, 45, 301, 77, 12]                       # one placeholder per image
    double = [3] + [IMG_TOK] * 4 + [40, 41] + [IMG_TOK] * 4 + [60, 61, 62]
    sp = SamplingParams(max_tokens=6, temperature=0.0, ignore_eos=True)
    outs = llm.generate([
        {"prompt_token_ids": expanded, "multi_modal_data": {"image": img_a}},
        {"prompt_token_ids": short, "multi_modal_data": {"image": img_b}},          # same text, other image
        {"prompt_token_ids": double, "multi_modal_data": {"pixel_values": two}},
        {"prompt_token_ids": [5, 9, 33, 100, 7]},                                     # text only, same batch
    ], sp)
    got = [list(o.outputs[0].token_ids) for o in outs]
    assert got[0] == _want(hf, expanded, img_a)
    assert got[1] == _want(hf, expanded, img_b)
    assert got[2] == _want(hf, double, two)
    with torch.no_grad():
        text = hf.generate(input_ids=torch.tensor([[5, 9, 33, 100, 7]]), max_new_tokens=6, do_sample=False,
                           eos_token_id=None, pad_token_id=0)[0, 5:].tolist()
    assert got[3] == text
    # the same prompt with another image must not reuse the first image's cached blocks (and gives its own answer)
    again = llm.generate([{"prompt_token_ids": expanded, "multi_modal_data": {"image": img_b}}], sp)
    assert list(again[0].outputs[0].token_ids) == got[1]


def test_placeholder_count_is_checked(tmp_path):
    from vllm_metax_b200 import LLM, SamplingParams

    _hf_llava(tmp_path)
    llm = LLM(str(tmp_path), dtype="float32", device="cpu", max_model_len=128, num_gpu_blocks=16, block_size=16)
    with pytest.raises(ValueError, match="placeholder"):
        llm.generate([{"prompt_token_ids": [1, 2, 3], "multi_modal_data": {"image": torch.zeros(1, 3, 28, 28)}}],
                     SamplingParams(max_tokens=2))
    img = torch.randint(0, 255, (3, 50, 40), dtype=torch.uint8)          # raw image: resized + normalised here
    out = llm.generate([{"prompt_token_ids": [1, IMG_TOK, 3], "multi_modal_data": {"image": img}}],
                       SamplingParams(max_tokens=2, ignore_eos=True))
    assert len(out[0].outputs[0].token_ids) == 2


def test_chat_completion_with_image_over_http(tmp_path):
    """An OpenAI chat request with a base64 image part: the server decodes it, places the model's placeholder token
    where the image stands in the rendered prompt, and the answer equals the offline call with the same inputs."""
    import asyncio
    import base64
    import io
    import json

    httpx = pytest.importorskip("httpx")
    from PIL import Image

    from vllm_metax_b200 import LLM, SamplingParams
    from vllm_metax_b200.entrypoints.async_engine import AsyncLLM
    from vllm_metax_b200.entrypoints.openai_server import build_app

    class Tok:
        chat_template = None

        def encode(self, text, add_special_tokens=True):
            return [3 + (ord(c) % 200) for c in text][:48] or [3]

        def decode(self, ids, skip_special_tokens=True):
            return "".join(chr(97 + (i % 26)) for i in ids)

    _hf_llava(tmp_path)
    llm = LLM(str(tmp_path), dtype="float32", device="cpu", max_model_len=128, num_gpu_blocks=32, block_size=16, tokenizer=Tok())
    img = Image.fromarray((torch.rand(40, 30, 3) * 255).to(torch.uint8).numpy())
    buf = io.BytesIO()
    img.save(buf, format="PNG")
    url = "data:image/png;base64," + base64.b64encode(buf.getvalue()).decode()
    body = {"model": "llava", "max_tokens": 5, "messages": [{"role": "user", "content": [
        {"type": "text", "text": "look: "}, {"type": "image_url", "image_url": {"url": url}}, {"type": "text", "text": " what?"}]}]}
    allm = AsyncLLM(llm)
    app = build_app(allm, "llava")

    async def go(b):
        async with httpx.AsyncClient(transport=httpx.ASGITransport(app=app), base_url="http://t") as c:
            r = await c.post("/v1/chat/completions", json=b)
            return r.status_code, r.text
    try:
        code, text = asyncio.run(go(body))
        assert code == 200, text
        answer = json.loads(text)["choices"][0]["message"]["content"]
        assert json.loads(text)["usage"]["prompt_tokens"] > 4                  # the image run is part of the prompt
        # same request offline: the prompt text around the image, placeholder in between
        from vllm_metax_b200.entrypoints.openai_server import render_chat

        rendered = render_chat(Tok(), [{"role": "user", "content": "look: @@ what?"}])
        left, right = rendered.split("@@")
        ids = Tok().encode(left) + [IMG_TOK] + Tok().encode(right)
        code2, text2 = asyncio.run(go(dict(body, messages=[{"role": "user", "content": [
            {"type": "image_url", "image_url": {"url": "http://example.com/x.png"}}]}])))
        assert code2 == 400 and "data:" in text2
    finally:
        allm.shutdown()
    off = llm.generate([{"prompt_token_ids": ids, "multi_modal_data": {"image": img}}],
                       SamplingParams(max_tokens=5, temperature=0.0))
    assert Tok().decode(off[0].outputs[0].token_ids) == answer


def test_internvl_matches_hugging_face(tmp_path):
    """InternViT tower (layer scale, no pre-norm) + pixel-shuffle + LayerNorm projector over a Qwen2 decoder."""
    from vllm_metax_b200 import LLM, SamplingParams

    torch.manual_seed(0)
    vc = tf.InternVLVisionConfig(hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4,
                                 image_size=[56, 56], patch_size=[14, 14])
    tc = tf.Qwen2Config(vocab_size=512, hidden_size=128, intermediate_size=256, num_hidden_layers=2, num_attention_heads=4,
                        num_key_value_heads=2, max_position_embeddings=256)
    c = tf.InternVLConfig(vision_config=vc, text_config=tc, image_token_id=IMG_TOK, image_seq_length=4)
    hf = tf.InternVLForConditionalGeneration(c).eval().float()
    with torch.no_grad():
        for p in hf.parameters():
            if p.dim() == 1:
                p.add_(0.1 * torch.randn_like(p))
            else:
                p.mul_(3.0)
    hf.save_pretrained(str(tmp_path))
    llm = LLM(str(tmp_path), dtype="float32", device="cpu", max_model_len=128, num_gpu_blocks=32, block_size=16,
              max_num_batched_tokens=6)
    assert llm.engine.runner.model.tokens_per_image == 4            # 4 x 4 patches folded 2 x 2
    g = torch.Generator().manual_seed(2)
    img = torch.randn(1, 3, 56, 56, generator=g)
    ids = [5, 9] + [IMG_TOK] * 4 + [33, 100, 7, 8, 200, 31, 2]
    out = llm.generate([{"prompt_token_ids": [5, 9, IMG_TOK, 33, 100, 7, 8, 200, 31, 2], "multi_modal_data": {"image": img}}],
                       SamplingParams(max_tokens=6, temperature=0.0, ignore_eos=True))
    assert list(out[0].outputs[0].token_ids) == _want(hf, ids, img)


def test_internvl_chat_original_export(tmp_path):
    """The original InternVL tensor names (fused ``attn.qkv``, ``ls1`` / ``ls2``, ``mlp1.*``, ``llm_config``) load onto
    the same graph: a Hugging Face InternVL model rewritten into that dialect must give the Hugging Face answer."""
    import json

    from safetensors.torch import save_file

    from vllm_metax_b200 import LLM, SamplingParams

    torch.manual_seed(3)
    vc = tf.InternVLVisionConfig(hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4,
                                 image_size=[56, 56], patch_size=[14, 14], attention_bias=True)
    tc = tf.Qwen2Config(vocab_size=512, hidden_size=128, intermediate_size=256, num_hidden_layers=2, num_attention_heads=4,
                        num_key_value_heads=2, max_position_embeddings=256, tie_word_embeddings=False)
    hf = tf.InternVLForConditionalGeneration(tf.InternVLConfig(vision_config=vc, text_config=tc, image_token_id=IMG_TOK,
                                                               image_seq_length=4, tie_word_embeddings=False)).eval().float()
    with torch.no_grad():
        for p in hf.parameters():
            p.add_(0.1 * torch.randn_like(p)) if p.dim() == 1 else p.mul_(3.0)
    sd, out = hf.state_dict(), {}
    for k, v in sd.items():
        if k.startswith("model.language_model."):
            out["language_model.model." + k[len("model.language_model."):]] = v
        elif k == "lm_head.weight":
            out["language_model.lm_head.weight"] = v
        elif k.startswith("model.multi_modal_projector."):
            n = k[len("model.multi_modal_projector."):]
            out["mlp1." + n.replace("layer_norm", "0").replace("linear_1", "1").replace("linear_2", "3")] = v
        elif k.startswith("model.vision_tower.embeddings."):
            n = k.rsplit(".", 1)[1] if "patch_embeddings" in k else k[len("model.vision_tower.embeddings."):]
            name = {"cls_token": "class_embedding", "position_embeddings": "position_embedding", "weight": "patch_embedding.weight",
                    "bias": "patch_embedding.bias"}[n]
            out["vision_model.embeddings." + name] = v
    for i in range(2):
        pre, dst = f"model.vision_tower.encoder.layer.{i}.", f"vision_model.encoder.layers.{i}."
        for kind in ("weight", "bias"):
            out[dst + f"attn.qkv.{kind}"] = torch.cat([sd[pre + f"attention.{x}_proj.{kind}"] for x in "qkv"], 0)
            out[dst + f"attn.proj.{kind}"] = sd[pre + f"attention.projection_layer.{kind}"]
            out[dst + f"norm1.{kind}"] = sd[pre + f"layernorm_before.{kind}"]
            out[dst + f"norm2.{kind}"] = sd[pre + f"layernorm_after.{kind}"]
            out[dst + f"mlp.fc1.{kind}"] = sd[pre + f"mlp.fc1.{kind}"]
            out[dst + f"mlp.fc2.{kind}"] = sd[pre + f"mlp.fc2.{kind}"]
        out[dst + "ls1"], out[dst + "ls2"] = sd[pre + "lambda_1"], sd[pre + "lambda_2"]
    save_file({k: v.contiguous() for k, v in out.items()}, str(tmp_path / "model.safetensors"))
    cfg = {"architectures": ["InternVLChatModel"], "downsample_ratio": 0.5, "select_layer": -1, "img_context_token_id": IMG_TOK,
           "vision_config": {"hidden_size": 64, "intermediate_size": 128, "num_hidden_layers": 2, "num_attention_heads": 4,
                             "image_size": 56, "patch_size": 14, "qkv_bias": True, "hidden_act": "gelu", "layer_norm_eps": 1e-6,
                             "norm_type": "layer_norm"},
           "llm_config": dict(tc.to_dict(), architectures=["Qwen2ForCausalLM"]), "torch_dtype": "float32"}
    (tmp_path / "config.json").write_text(json.dumps(cfg))
    llm = LLM(str(tmp_path), dtype="float32", device="cpu", max_model_len=128, num_gpu_blocks=32, block_size=16)
    img = torch.randn(1, 3, 56, 56, generator=torch.Generator().manual_seed(4))
    ids = [5, 9] + [IMG_TOK] * 4 + [33, 100, 7, 8, 200, 31, 2]
    got = llm.generate([{"prompt_token_ids": ids, "multi_modal_data": {"image": img}}],
                       SamplingParams(max_tokens=6, temperature=0.0, ignore_eos=True))
    assert list(got[0].outputs[0].token_ids) == _want(hf, ids, img)


# ------------------------------------------------------------------ Qwen2-VL: dynamic-resolution tower + M-RoPE
QV_IMG, QV_START, QV_END = 500, 501, 502


def _hf_qwen2vl(tmp_path):
    torch.manual_seed(0)
    c = tf.Qwen2VLConfig(
        text_config=dict(vocab_size=512, hidden_size=128, intermediate_size=256, num_hidden_layers=2, num_attention_heads=4,
                         num_key_value_heads=2, max_position_embeddings=256, tie_word_embeddings=False,
                         rope_parameters={"rope_type": "default", "rope_theta": 10000.0, "mrope_section": [4, 6, 6]}),
        vision_config=dict(depth=2, embed_dim=64, hidden_size=128, num_heads=4, mlp_ratio=2, in_channels=3, patch_size=14,
                           spatial_merge_size=2, temporal_patch_size=2),
        image_token_id=QV_IMG, video_token_id=503, vision_start_token_id=QV_START, vision_end_token_id=QV_END)
    hf = tf.Qwen2VLForConditionalGeneration(c).eval().float()
    with torch.no_grad():
        for p in hf.parameters():
            if p.dim() == 1:
                p.add_(0.1 * torch.randn_like(p))
            else:
                p.mul_(2.0)
    hf.save_pretrained(str(tmp_path))
    return hf


@pytest.mark.parametrize("chunk", [64, 7])
def test_qwen2_vl_matches_hugging_face(tmp_path, chunk):
    from vllm_metax_b200 import LLM, SamplingParams

    hf = _hf_qwen2vl(tmp_path)
    llm = LLM(str(tmp_path), dtype="float32", device="cpu", max_model_len=128, num_gpu_blocks=32, block_size=16,
              max_num_batched_tokens=chunk)
    assert llm.engine.runner.uses_mrope
    g = torch.Generator().manual_seed(1)
    grid_a, grid_b = (1, 4, 6), (1, 2, 4)                      # patches; 6 and 2 tokens after the 2 x 2 merge
    pa, pb = torch.randn(24, 1176, generator=g), torch.randn(8, 1176, generator=g)
    one = [5, 9, QV_START] + [QV_IMG] * 6 + [QV_END, 33, 100, 7, 8, 200, 31]
    two = [3, QV_START] + [QV_IMG] * 6 + [QV_END, 40, QV_START] + [QV_IMG] * 2 + [QV_END, 60, 61, 62]
    short = [5, 9, QV_START, QV_IMG, QV_END, 33, 100, 7, 8, 200, 31]          # one placeholder for the image
    sp = SamplingParams(max_tokens=6, temperature=0.0, ignore_eos=True)
    outs = llm.generate([
        {"prompt_token_ids": one, "multi_modal_data": {"pixel_values": pa, "image_grid_thw": [grid_a]}},
        {"prompt_token_ids": two, "multi_modal_data": {"pixel_values": torch.cat([pa, pb]), "image_grid_thw": [grid_a, grid_b]}},
        {"prompt_token_ids": short, "multi_modal_data": {"pixel_values": pa, "image_grid_thw": [grid_a]}},
        {"prompt_token_ids": [5, 9, 33, 100, 7]},
    ], sp)
    got = [list(o.outputs[0].token_ids) for o in outs]

    def want(ids, pixels=None, grids=None):
        kw = {} if pixels is None else dict(pixel_values=pixels, image_grid_thw=torch.tensor(grids))
        with torch.no_grad():
            out = hf.generate(input_ids=torch.tensor([ids]), max_new_tokens=6, do_sample=False, eos_token_id=None,
                              pad_token_id=0, **kw)
        return out[0, len(ids):].tolist()

    assert got[0] == want(one, pa, [grid_a])
    assert got[1] == want(two, torch.cat([pa, pb]), [grid_a, grid_b])
    assert got[2] == got[0]
    assert got[3] == want([5, 9, 33, 100, 7])


def test_mrope_prompt_table():
    from vllm_metax_b200.models.qwen2_vl import mrope_prompt_positions

    ids = [1, 2, QV_IMG, QV_IMG, QV_IMG, QV_IMG, QV_IMG, QV_IMG, 3, 4]
    pos, delta = mrope_prompt_positions(ids, [(1, 4, 6)], QV_IMG, 2)          # 2 x 3 merged grid
    assert pos[:, :2].tolist() == [[0, 1]] * 3
    assert pos[0, 2:8].tolist() == [2] * 6
    assert pos[1, 2:8].tolist() == [2, 2, 2, 3, 3, 3] and pos[2, 2:8].tolist() == [2, 3, 4, 2, 3, 4]
    assert pos[:, 8:].tolist() == [[5, 6]] * 3 and delta == 7 - 10


def test_qwen2_5_vl_matches_hugging_face(tmp_path):
    """Qwen2.5-VL: RMSNorm + SiLU-gated vision blocks, window attention with one full-attention block, RMSNorm merger."""
    from vllm_metax_b200 import LLM, SamplingParams

    torch.manual_seed(0)
    c = tf.Qwen2_5_VLConfig(
        text_config=dict(vocab_size=512, hidden_size=128, intermediate_size=256, num_hidden_layers=2, num_attention_heads=4,
                         num_key_value_heads=2, max_position_embeddings=256, tie_word_embeddings=False,
                         rope_parameters={"rope_type": "default", "rope_theta": 10000.0, "mrope_section": [4, 6, 6]}),
        vision_config=dict(depth=3, hidden_size=64, intermediate_size=96, out_hidden_size=128, num_heads=4, in_channels=3,
                           patch_size=14, spatial_merge_size=2, temporal_patch_size=2, window_size=56,
                           fullatt_block_indexes=[1]),
        image_token_id=QV_IMG, video_token_id=503, vision_start_token_id=QV_START, vision_end_token_id=QV_END)
    hf = tf.Qwen2_5_VLForConditionalGeneration(c).eval().float()
    with torch.no_grad():
        for p in hf.parameters():
            if p.dim() == 1:
                p.add_(0.1 * torch.randn_like(p))
            else:
                p.mul_(2.0)
    hf.save_pretrained(str(tmp_path))
    llm = LLM(str(tmp_path), dtype="float32", device="cpu", max_model_len=128, num_gpu_blocks=32, block_size=16,
              max_num_batched_tokens=64)
    g = torch.Generator().manual_seed(1)
    grid = (1, 6, 8)                                           # 3 x 4 merge units, windows of 2 x 2 units: ragged edges
    px = torch.randn(48, 1176, generator=g)
    ids = [5, 9, QV_START] + [QV_IMG] * 12 + [QV_END, 33, 100, 7, 8]
    sp = SamplingParams(max_tokens=6, temperature=0.0, ignore_eos=True)
    got = list(llm.generate([{"prompt_token_ids": ids, "multi_modal_data": {"pixel_values": px, "image_grid_thw": [grid]}}],
                            sp)[0].outputs[0].token_ids)
    with torch.no_grad():
        out = hf.generate(input_ids=torch.tensor([ids]), pixel_values=px, image_grid_thw=torch.tensor([grid]),
                          mm_token_type_ids=torch.tensor([[1 if t == QV_IMG else 0 for t in ids]]),
                          max_new_tokens=6, do_sample=False, eos_token_id=None, pad_token_id=0)
    assert got == out[0, len(ids):].tolist()


def test_llava_next_matches_hugging_face(tmp_path):
    """Any-resolution LLaVA: base image + tile grid, unpadded feature map, newline column; wide, tall and small
    images (different grids and different token counts) against Hugging Face's model on the same pixel tensors."""
    from vllm_metax_b200 import LLM, SamplingParams
    from vllm_metax_b200.models.llava import select_best_resolution

    torch.manual_seed(0)
    vc = tf.CLIPVisionConfig(hidden_size=64, intermediate_size=128, num_hidden_layers=3, num_attention_heads=4,
                             image_size=28, patch_size=14, projection_dim=32)
    tc = tf.LlamaConfig(vocab_size=512, hidden_size=128, intermediate_size=256, num_hidden_layers=2, num_attention_heads=4,
                        num_key_value_heads=2, max_position_embeddings=256)
    pins = [[28, 56], [56, 28], [56, 56], [28, 84], [84, 28]]
    c = tf.LlavaNextConfig(vision_config=vc, text_config=tc, image_token_index=IMG_TOK, vision_feature_layer=-2,
                           vision_feature_select_strategy="default", image_grid_pinpoints=pins, image_seq_length=4)
    hf = tf.LlavaNextForConditionalGeneration(c).eval().float()
    with torch.no_grad():
        for p in hf.parameters():
            if p.dim() == 1:
                p.add_(0.1 * torch.randn_like(p))
            else:
                p.mul_(3.0)
    hf.save_pretrained(str(tmp_path))
    llm = LLM(str(tmp_path), dtype="float32", device="cpu", max_model_len=160, num_gpu_blocks=40, block_size=16,
              max_num_batched_tokens=24)
    model = llm.engine.runner.model
    assert type(model).__name__ == "LlavaNextForConditionalGeneration" and float(model.image_newline.abs().sum()) > 0
    g = torch.Generator().manual_seed(2)
    sp = SamplingParams(max_tokens=5, temperature=0.0, ignore_eos=True)
    for hw in [(30, 100), (90, 40), (50, 50), (20, 20)]:
        ch, cw = select_best_resolution(hw, [tuple(p) for p in pins])
        tiles = 1 + (ch // 28) * (cw // 28)
        pixels = torch.randn(1, tiles, 3, 28, 28, generator=g)
        sizes = torch.tensor([list(hw)])
        with torch.no_grad():       # Hugging Face checks the count itself: a wrong one fails its generate call below
            n_tok = model.pack_features(model.embed_multimodal(pixels[0]), hw).shape[0]
        ids = [5, 9] + [IMG_TOK] * n_tok + [33, 100, 7, 8]
        with torch.no_grad():
            want = hf.generate(input_ids=torch.tensor([ids]), pixel_values=pixels, image_sizes=sizes, max_new_tokens=5,
                               do_sample=False, eos_token_id=None, pad_token_id=0)[0, len(ids):].tolist()
        out = llm.generate([{"prompt_token_ids": [5, 9, IMG_TOK, 33, 100, 7, 8],
                             "multi_modal_data": {"pixel_values": pixels, "image_sizes": sizes}}], sp)
        assert len(out[0].prompt_token_ids) == len(ids), (hw, n_tok)
        assert list(out[0].outputs[0].token_ids) == want, hw
    # raw images go through this package's own tiling
    img = torch.randint(0, 255, (3, 40, 100), dtype=torch.uint8)
    out = llm.generate([{"prompt_token_ids": [1, IMG_TOK, 3], "multi_modal_data": {"image": img}}], sp)
    assert len(out[0].outputs[0].token_ids) == 5


@pytest.mark.parametrize("chunk", [64, 7])
def test_qwen3_vl_matches_hugging_face(tmp_path, chunk):
    """Qwen3-VL: interpolated position embeddings, interleaved M-RoPE, DeepStack features added after the first
    decoder layers - across chunked prefill (the image run is split between steps) against Hugging Face."""
    from vllm_metax_b200 import LLM, SamplingParams

    torch.manual_seed(0)
    c = tf.Qwen3VLConfig(
        text_config=dict(vocab_size=512, hidden_size=128, intermediate_size=256, num_hidden_layers=3, num_attention_heads=4,
                         num_key_value_heads=2, head_dim=32, max_position_embeddings=256, tie_word_embeddings=False,
                         rope_parameters={"rope_type": "default", "rope_theta": 10000.0, "mrope_section": [6, 5, 5],
                                          "mrope_interleaved": True}),
        vision_config=dict(depth=3, hidden_size=64, intermediate_size=96, out_hidden_size=128, num_heads=4, in_channels=3,
                           patch_size=8, spatial_merge_size=2, temporal_patch_size=2, num_position_embeddings=36,
                           deepstack_visual_indexes=[0, 1]),
        image_token_id=QV_IMG, video_token_id=503, vision_start_token_id=QV_START, vision_end_token_id=QV_END,
        tie_word_embeddings=False)
    hf = tf.Qwen3VLForConditionalGeneration(c).eval().float()
    with torch.no_grad():
        for p in hf.parameters():
            if p.dim() == 1:
                p.add_(0.1 * torch.randn_like(p))
            else:
                p.mul_(2.0)
    hf.save_pretrained(str(tmp_path))
    llm = LLM(str(tmp_path), dtype="float32", device="cpu", max_model_len=128, num_gpu_blocks=32, block_size=16,
              max_num_batched_tokens=chunk)
    model = llm.engine.runner.model
    assert type(model).__name__ == "Qwen3VLForConditionalGeneration" and model.language_model.model.takes_deepstack
    g = torch.Generator().manual_seed(1)
    grid_a, grid_b = (1, 4, 6), (1, 2, 4)
    dim = 3 * 2 * 8 * 8
    pa, pb = torch.randn(24, dim, generator=g), torch.randn(8, dim, generator=g)
    one = [5, 9, QV_START] + [QV_IMG] * 6 + [QV_END, 33, 100, 7, 8, 200, 31]
    two = [3, QV_START] + [QV_IMG] * 6 + [QV_END, 40, QV_START] + [QV_IMG] * 2 + [QV_END, 60, 61, 62]
    sp = SamplingParams(max_tokens=6, temperature=0.0, ignore_eos=True)
    outs = llm.generate([
        {"prompt_token_ids": one, "multi_modal_data": {"pixel_values": pa, "image_grid_thw": [grid_a]}},
        {"prompt_token_ids": two, "multi_modal_data": {"pixel_values": torch.cat([pa, pb]), "image_grid_thw": [grid_a, grid_b]}},
        {"prompt_token_ids": [5, 9, 33, 100, 7]},
    ], sp)
    got = [list(o.outputs[0].token_ids) for o in outs]

    def want(ids, pixels=None, grids=None):
        kw = {} if pixels is None else dict(pixel_values=pixels, image_grid_thw=torch.tensor(grids),
                                            mm_token_type_ids=torch.tensor([[1 if t == QV_IMG else 0 for t in ids]]))
        with torch.no_grad():
            out = hf.generate(input_ids=torch.tensor([ids]), max_new_tokens=6, do_sample=False, eos_token_id=None,
                              pad_token_id=0, **kw)
        return out[0, len(ids):].tolist()

    assert got[0] == want(one, pa, [grid_a])
    assert got[1] == want(two, torch.cat([pa, pb]), [grid_a, grid_b])
    assert got[2] == want([5, 9, 33, 100, 7])


def test_mrope_frequency_streams():
    from vllm_metax_b200.models.qwen2_vl import mrope_stream_of_frequency

    assert mrope_stream_of_frequency([2, 3, 3], 8, False) == [0, 0, 1, 1, 1, 2, 2, 2]
    assert mrope_stream_of_frequency([6, 5, 5], 16, True) == [0, 1, 2] * 5 + [0]
    assert mrope_stream_of_frequency([24, 20, 20], 64, True)[58:] == [1, 2, 0, 0, 0, 0]


def test_qwen3_vl_moe_matches_hugging_face(tmp_path):
    """The same tower, M-RoPE and DeepStack over the mixture-of-experts decoder; stacked expert tensors of the
    checkpoint are split per expert at load."""
    from vllm_metax_b200 import LLM, SamplingParams

    torch.manual_seed(0)
    c = tf.Qwen3VLMoeConfig(
        text_config=dict(vocab_size=512, hidden_size=128, intermediate_size=256, num_hidden_layers=3, num_attention_heads=4,
                         num_key_value_heads=2, head_dim=32, max_position_embeddings=256, num_experts=4, num_experts_per_tok=2,
                         moe_intermediate_size=64, decoder_sparse_step=1, mlp_only_layers=[], tie_word_embeddings=False,
                         rope_parameters={"rope_type": "default", "rope_theta": 10000.0, "mrope_section": [6, 5, 5],
                                          "mrope_interleaved": True}),
        vision_config=dict(depth=2, hidden_size=64, intermediate_size=96, out_hidden_size=128, num_heads=4, in_channels=3,
                           patch_size=8, spatial_merge_size=2, temporal_patch_size=2, num_position_embeddings=36,
                           deepstack_visual_indexes=[0, 1]),
        image_token_id=QV_IMG, video_token_id=503, vision_start_token_id=QV_START, vision_end_token_id=QV_END,
        tie_word_embeddings=False)
    hf = tf.Qwen3VLMoeForConditionalGeneration(c).eval().float()
    with torch.no_grad():
        for p in hf.parameters():
            if p.dim() == 1:
                p.add_(0.1 * torch.randn_like(p))
            elif p.dim() == 3:
                p.normal_(0, 0.15)                       # stacked experts (left uninitialised by the constructor)
            else:
                p.mul_(2.0)
    hf.save_pretrained(str(tmp_path))
    llm = LLM(str(tmp_path), dtype="float32", device="cpu", max_model_len=128, num_gpu_blocks=32, block_size=16,
              max_num_batched_tokens=9)
    assert type(llm.engine.runner.model).__name__ == "Qwen3VLMoeForConditionalGeneration"
    g = torch.Generator().manual_seed(3)
    grid = (1, 4, 4)
    px = torch.randn(16, 3 * 2 * 8 * 8, generator=g)
    ids = [5, 9, QV_START] + [QV_IMG] * 4 + [QV_END, 33, 100, 7, 8, 200, 31]
    sp = SamplingParams(max_tokens=6, temperature=0.0, ignore_eos=True)
    got = llm.generate([{"prompt_token_ids": ids, "multi_modal_data": {"pixel_values": px, "image_grid_thw": [grid]}},
                        {"prompt_token_ids": [5, 9, 33, 100, 7]}], sp)
    with torch.no_grad():
        want = hf.generate(input_ids=torch.tensor([ids]), max_new_tokens=6, do_sample=False, eos_token_id=None, pad_token_id=0,
                           pixel_values=px, image_grid_thw=torch.tensor([grid]),
                           mm_token_type_ids=torch.tensor([[1 if t == QV_IMG else 0 for t in ids]]))[0, len(ids):].tolist()
        text = hf.generate(input_ids=torch.tensor([[5, 9, 33, 100, 7]]), max_new_tokens=6, do_sample=False, eos_token_id=None,
                           pad_token_id=0)[0, 5:].tolist()
    assert list(got[0].outputs[0].token_ids) == want
    assert list(got[1].outputs[0].token_ids) == text


@pytest.mark.parametrize("chunk", [64, 7])
def test_glm4v_matches_hugging_face(tmp_path, chunk):
    """GLM-4.1V: bicubically sampled position embeddings, RMSNorm / SwiGLU vision blocks, convolutional patch merge,
    gated merger; GLM-4 decoder with M-RoPE over the rotated half of every head in adjacent pairs."""
    from vllm_metax_b200 import LLM, SamplingParams

    torch.manual_seed(0)
    c = tf.Glm4vConfig(
        text_config=dict(vocab_size=512, hidden_size=128, intermediate_size=256, num_hidden_layers=2, num_attention_heads=4,
                         num_key_value_heads=2, head_dim=32, max_position_embeddings=256, tie_word_embeddings=False,
                         rope_parameters={"rope_type": "default", "rope_theta": 10000.0, "mrope_section": [2, 3, 3],
                                          "partial_rotary_factor": 0.5}),
        vision_config=dict(depth=2, hidden_size=64, intermediate_size=96, out_hidden_size=128, num_heads=4, in_channels=3,
                           patch_size=8, spatial_merge_size=2, temporal_patch_size=2, image_size=48, attention_bias=False),
        image_token_id=QV_IMG, video_token_id=503, image_start_token_id=QV_START, image_end_token_id=QV_END,
        tie_word_embeddings=False)
    hf = tf.Glm4vForConditionalGeneration(c).eval().float()
    with torch.no_grad():
        for p in hf.parameters():
            if p.dim() == 1:
                p.add_(0.1 * torch.randn_like(p))
            else:
                p.mul_(2.0)
    hf.save_pretrained(str(tmp_path))
    llm = LLM(str(tmp_path), dtype="float32", device="cpu", max_model_len=128, num_gpu_blocks=32, block_size=16,
              max_num_batched_tokens=chunk)
    assert type(llm.engine.runner.model).__name__ == "Glm4vForConditionalGeneration" and llm.engine.runner.uses_mrope
    g = torch.Generator().manual_seed(1)
    grid_a, grid_b = (1, 4, 6), (1, 2, 4)
    dim = 3 * 2 * 8 * 8
    pa, pb = torch.randn(24, dim, generator=g), torch.randn(8, dim, generator=g)
    one = [5, 9, QV_START] + [QV_IMG] * 6 + [QV_END, 33, 100, 7, 8, 200, 31]
    two = [3, QV_START] + [QV_IMG] * 6 + [QV_END, 40, QV_START] + [QV_IMG] * 2 + [QV_END, 60, 61, 62]
    sp = SamplingParams(max_tokens=6, temperature=0.0, ignore_eos=True)
    outs = llm.generate([
        {"prompt_token_ids": one, "multi_modal_data": {"pixel_values": pa, "image_grid_thw": [grid_a]}},
        {"prompt_token_ids": two, "multi_modal_data": {"pixel_values": torch.cat([pa, pb]), "image_grid_thw": [grid_a, grid_b]}},
        {"prompt_token_ids": [5, 9, 33, 100, 7]},
    ], sp)
    got = [list(o.outputs[0].token_ids) for o in outs]

    def want(ids, pixels=None, grids=None):
        kw = {} if pixels is None else dict(pixel_values=pixels, image_grid_thw=torch.tensor(grids),
                                            mm_token_type_ids=torch.tensor([[1 if t == QV_IMG else 0 for t in ids]]))
        with torch.no_grad():
            out = hf.generate(input_ids=torch.tensor([ids]), max_new_tokens=6, do_sample=False, eos_token_id=None,
                              pad_token_id=0, **kw)
        return out[0, len(ids):].tolist()

    assert got[0] == want(one, pa, [grid_a])
    assert got[1] == want(two, torch.cat([pa, pb]), [grid_a, grid_b])
    assert got[2] == want([5, 9, 33, 100, 7])
    assert len(set(got[0])) > 1 or len(set(got[1])) > 1           # not a degenerate constant continuation


def test_glm4v_moe_matches_hugging_face(tmp_path):
    """GLM-4.5V: the GLM-4.1V tower over the GLM-4.5 mixture-of-experts decoder (sigmoid routing with bias correction,
    shared expert, a dense first layer), stacked expert tensors split at load."""
    from vllm_metax_b200 import LLM, SamplingParams

    torch.manual_seed(0)
    c = tf.Glm4vMoeConfig(
        text_config=dict(vocab_size=512, hidden_size=128, intermediate_size=256, num_hidden_layers=3, num_attention_heads=4,
                         num_key_value_heads=2, head_dim=32, max_position_embeddings=256, tie_word_embeddings=False,
                         n_routed_experts=8, num_experts_per_tok=2, moe_intermediate_size=64, n_shared_experts=1, n_group=1,
                         topk_group=1, first_k_dense_replace=1, norm_topk_prob=True, routed_scaling_factor=1.0,
                         use_qk_norm=False,
                         rope_parameters={"rope_type": "default", "rope_theta": 10000.0, "mrope_section": [2, 3, 3],
                                          "partial_rotary_factor": 0.5}),
        vision_config=dict(depth=2, hidden_size=64, intermediate_size=96, out_hidden_size=128, num_heads=4, in_channels=3,
                           patch_size=8, spatial_merge_size=2, temporal_patch_size=2, image_size=48, attention_bias=False),
        image_token_id=QV_IMG, video_token_id=503, image_start_token_id=QV_START, image_end_token_id=QV_END,
        tie_word_embeddings=False)
    hf = tf.Glm4vMoeForConditionalGeneration(c).eval().float()
    with torch.no_grad():
        for p in hf.parameters():
            if p.dim() == 1:
                p.add_(0.1 * torch.randn_like(p))
            elif p.dim() == 3:
                p.normal_(0, 0.15)
            else:
                p.mul_(2.0)
    hf.save_pretrained(str(tmp_path))
    llm = LLM(str(tmp_path), dtype="float32", device="cpu", max_model_len=128, num_gpu_blocks=32, block_size=16,
              max_num_batched_tokens=9)
    assert type(llm.engine.runner.model).__name__ == "Glm4vMoeForConditionalGeneration"
    assert llm.engine.cfg.model.scoring_func == "sigmoid"
    g = torch.Generator().manual_seed(1)
    grid = (1, 4, 6)
    px = torch.randn(24, 3 * 2 * 8 * 8, generator=g)
    ids = [5, 9, QV_START] + [QV_IMG] * 6 + [QV_END, 33, 100, 7, 8, 200, 31]
    sp = SamplingParams(max_tokens=5, temperature=0.0, ignore_eos=True)
    got = llm.generate([{"prompt_token_ids": ids, "multi_modal_data": {"pixel_values": px, "image_grid_thw": [grid]}},
                        {"prompt_token_ids": [5, 9, 33, 100, 7]}], sp)
    with torch.no_grad():
        want = hf.generate(input_ids=torch.tensor([ids]), max_new_tokens=5, do_sample=False, eos_token_id=None, pad_token_id=0,
                           pixel_values=px, image_grid_thw=torch.tensor([grid]),
                           mm_token_type_ids=torch.tensor([[1 if t == QV_IMG else 0 for t in ids]]))[0, len(ids):].tolist()
        text = hf.generate(input_ids=torch.tensor([[5, 9, 33, 100, 7]]), max_new_tokens=5, do_sample=False, eos_token_id=None,
                           pad_token_id=0)[0, 5:].tolist()
    assert list(got[0].outputs[0].token_ids) == want
    assert list(got[1].outputs[0].token_ids) == text


def test_llava_onevision_matches_hugging_face(tmp_path):
    """LLaVA-OneVision: SigLIP tower (no class token), any-resolution packing, and the bilinear shrink of feature maps
    larger than ``anyres_max_N`` tower images (forced here with N = 1)."""
    from vllm_metax_b200 import LLM, SamplingParams
    from vllm_metax_b200.models.llava import select_best_resolution

    torch.manual_seed(0)
    vc = tf.SiglipVisionConfig(hidden_size=64, intermediate_size=128, num_hidden_layers=3, num_attention_heads=4,
                               image_size=28, patch_size=14)
    tc = tf.Qwen2Config(vocab_size=512, hidden_size=128, intermediate_size=256, num_hidden_layers=2, num_attention_heads=4,
                        num_key_value_heads=2, max_position_embeddings=256, tie_word_embeddings=False)
    pins = [[28, 56], [56, 28], [56, 56], [28, 84], [84, 28]]
    c = tf.LlavaOnevisionConfig(vision_config=vc, text_config=tc, image_token_index=IMG_TOK, vision_feature_layer=-1,
                                vision_feature_select_strategy="full", image_grid_pinpoints=pins,
                                vision_aspect_ratio="anyres_max_1", tie_word_embeddings=False)
    hf = tf.LlavaOnevisionForConditionalGeneration(c).eval().float()
    with torch.no_grad():
        for p in hf.parameters():
            if p.dim() == 1:
                p.add_(0.1 * torch.randn_like(p))
            else:
                p.mul_(3.0)
    hf.save_pretrained(str(tmp_path))
    llm = LLM(str(tmp_path), dtype="float32", device="cpu", max_model_len=160, num_gpu_blocks=40, block_size=16,
              max_num_batched_tokens=24)
    model = llm.engine.runner.model
    assert type(model).__name__ == "LlavaOnevisionForConditionalGeneration" and model.max_tiles == 1
    g = torch.Generator().manual_seed(2)
    sp = SamplingParams(max_tokens=5, temperature=0.0, ignore_eos=True)
    shrunk = 0
    for hw in [(30, 100), (90, 40), (50, 50), (20, 20)]:
        ch, cw = select_best_resolution(hw, [tuple(p) for p in pins])
        tiles = 1 + (ch // 28) * (cw // 28)
        pixels = torch.randn(1, tiles, 3, 28, 28, generator=g)
        sizes = torch.tensor([list(hw)])
        with torch.no_grad():
            n_tok = model.pack_features(model.embed_multimodal(pixels[0]), hw).shape[0]
        shrunk += n_tok < 4 + (ch // 14) * (cw // 14 + 1) - 8                     # fewer tokens than the unshrunk map
        ids = [5, 9] + [IMG_TOK] * n_tok + [33, 100, 7, 8]
        with torch.no_grad():
            want = hf.generate(input_ids=torch.tensor([ids]), pixel_values=pixels, image_sizes=sizes, max_new_tokens=5,
                               do_sample=False, eos_token_id=None, pad_token_id=0)[0, len(ids):].tolist()
        out = llm.generate([{"prompt_token_ids": [5, 9, IMG_TOK, 33, 100, 7, 8],
                             "multi_modal_data": {"pixel_values": pixels, "image_sizes": sizes}}], sp)
        assert len(out[0].prompt_token_ids) == len(ids), (hw, n_tok)
        assert list(out[0].outputs[0].token_ids) == want, hw
    assert shrunk >= 1                                                            # the shrink path was exercised


def test_qwen2_vl_video_matches_hugging_face(tmp_path):
    """A video (three temporal patches) and an image in one prompt: the video's tokens take the video placeholder, the
    temporal stream of M-RoPE advances per temporal patch."""
    from vllm_metax_b200 import LLM, SamplingParams

    hf = _hf_qwen2vl(tmp_path)
    llm = LLM(str(tmp_path), dtype="float32", device="cpu", max_model_len=128, num_gpu_blocks=32, block_size=16,
              max_num_batched_tokens=11)
    VID = 503
    g = torch.Generator().manual_seed(4)
    vgrid, igrid = (3, 2, 4), (1, 4, 6)                       # 3 x (1 x 2) = 6 video tokens; 6 image tokens
    pv, pi = torch.randn(24, 1176, generator=g), torch.randn(24, 1176, generator=g)
    ids = [5, QV_START] + [VID] * 6 + [QV_END, 40, QV_START] + [QV_IMG] * 6 + [QV_END, 60, 61]
    short = [5, QV_START, VID, QV_END, 40, QV_START, QV_IMG, QV_END, 60, 61]
    sp = SamplingParams(max_tokens=6, temperature=0.0, ignore_eos=True)
    mm = {"pixel_values": pi, "image_grid_thw": [igrid], "pixel_values_videos": pv, "video_grid_thw": [vgrid]}
    got = llm.generate([{"prompt_token_ids": ids, "multi_modal_data": mm},
                        {"prompt_token_ids": short, "multi_modal_data": mm}], sp)
    tt = torch.tensor([[1 if t == QV_IMG else (2 if t == VID else 0) for t in ids]])
    with torch.no_grad():
        want = hf.generate(input_ids=torch.tensor([ids]), max_new_tokens=6, do_sample=False, eos_token_id=None, pad_token_id=0,
                           pixel_values=pi, image_grid_thw=torch.tensor([igrid]), pixel_values_videos=pv,
                           video_grid_thw=torch.tensor([vgrid]), mm_token_type_ids=tt)[0, len(ids):].tolist()
    assert list(got[0].outputs[0].token_ids) == want
    assert list(got[1].outputs[0].token_ids) == want and len(got[1].prompt_token_ids) == len(ids)
    with pytest.raises(ValueError):
        llm.generate([{"prompt_token_ids": [5, VID, VID, VID, 6], "multi_modal_data": mm}], sp)
