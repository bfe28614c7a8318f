"""Image + text prompts (LLaVA / InternVL checkpoints).

    python examples/multimodal_inference.py --model /path/to/llava-1.5-7b-hf --image photo.jpg

The prompt holds one image placeholder (``<image>`` for LLaVA); the engine expands it to the vision tower's token
count, runs the tower once per request and merges the features into the prefill.
"""
import argparse

from PIL import Image

from vllm_metax_b200 import LLM, SamplingParams


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", required=True)
    ap.add_argument("--image", required=True)
    ap.add_argument("--question", default="What is shown in this image?")
    a = ap.parse_args()
    llm = LLM(a.model, max_model_len=4096)
    tok, model = llm.tokenizer, llm.engine.runner.model
    marker = tok.decode([model.image_token_id])
    ids = tok.encode(f"USER: {marker}\n{a.question} ASSISTANT:")
    out = llm.generate([{"prompt_token_ids": ids, "multi_modal_data": {"image": Image.open(a.image)}}],
                       SamplingParams(max_tokens=128, temperature=0.0))
    print(out[0].outputs[0].text)


if __name__ == "__main__":
    main()
