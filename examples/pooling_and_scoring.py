"""Embeddings, pair scores and prompt classification from a decoder checkpoint.

    python examples/pooling_and_scoring.py --model /path/to/hf_model

``embed`` pools the final hidden states (last token by default, or the mean), ``score`` is the cosine similarity of
two pooled texts, ``classify`` compares the next-token logits of a few label tokens.
"""
import argparse

from vllm_metax_b200 import LLM


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", required=True)
    a = ap.parse_args()
    llm = LLM(a.model, max_model_len=512)
    texts = ["The capital of France is Paris.", "Paris is the French capital.", "GPUs multiply matrices quickly."]
    emb = llm.embed(texts, pooling="mean")
    print("embedding shape:", tuple(emb.shape))
    print("similarities to the first text:", [round(float(emb[0] @ emb[i]), 3) for i in range(len(texts))])
    print("pair scores:", llm.score(texts[0], texts[1:]))
    tok = llm.tokenizer
    labels = [" positive", " negative"]
    ids = [tok.encode(w, add_special_tokens=False)[0] for w in labels]
    probs = llm.classify(["Review: I loved this film. Sentiment:", "Review: A waste of two hours. Sentiment:"], ids)
    for row in probs:
        print({w: round(float(p), 3) for w, p in zip(labels, row)})


if __name__ == "__main__":
    main()
