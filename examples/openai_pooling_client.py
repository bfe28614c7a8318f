"""Embeddings, similarity scores, re-ranking and prompt scoring against a running server.

    b200-serve serve <model dir> --port 8000
    python examples/openai_pooling_client.py http://127.0.0.1:8000
"""
import json
import sys
import urllib.request

base = sys.argv[1] if len(sys.argv) > 1 else "http://127.0.0.1:8000"


def post(path: str, body: dict) -> dict:
    req = urllib.request.Request(base + path, json.dumps(body).encode(), {"Content-Type": "application/json"})
    with urllib.request.urlopen(req) as r:
        return json.loads(r.read())


emb = post("/v1/embeddings", {"input": ["a photo of a cat", "a picture of a kitten", "quarterly revenue report"]})
print(len(emb["data"]), "embeddings of", len(emb["data"][0]["embedding"]), "dimensions")

print(post("/score", {"text_1": "a photo of a cat", "text_2": ["a picture of a kitten", "quarterly revenue report"]})["data"])

ranked = post("/v1/rerank", {"query": "feline", "documents": ["dogs bark", "cats purr", "stocks fell"], "top_n": 2})
print([(r["index"], round(r["relevance_score"], 3)) for r in ranked["results"]])

# the request evaluation harnesses send to score a continuation: echo the prompt with its token log-probabilities
scored = post("/v1/completions", {"prompt": "The capital of France is Paris", "max_tokens": 0, "echo": True, "logprobs": 1})
print(sum(x for x in scored["choices"][0]["logprobs"]["token_logprobs"] if x is not None))
