"""Reasoning content and token log-probabilities over the OpenAI-compatible server.

    python -m vllm_metax_b200.entrypoints.cli serve /path/to/DeepSeek-R1-Distill-Qwen-7B --reasoning-parser deepseek_r1
    python examples/reasoning_and_logprobs_client.py

The answer arrives split into ``reasoning_content`` (the text between the think tags) and ``content``; the second
request asks for the log-probability of every generated token and its three most likely alternatives.
"""
import argparse
import json
import urllib.request


def post(url: str, body: dict) -> dict:
    req = urllib.request.Request(url, data=json.dumps(body).encode(), headers={"Content-Type": "application/json"})
    return json.loads(urllib.request.urlopen(req, timeout=600).read())


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--url", default="http://127.0.0.1:8000/v1/chat/completions")
    ap.add_argument("--model", default="b200-model")
    a = ap.parse_args()
    q = [{"role": "user", "content": "Which is larger, 9.11 or 9.8?"}]
    msg = post(a.url, {"model": a.model, "messages": q, "max_tokens": 1024})["choices"][0]["message"]
    print("reasoning:", (msg.get("reasoning_content") or "")[:600])
    print("answer:", msg.get("content"))
    out = post(a.url, {"model": a.model, "messages": q, "max_tokens": 8, "logprobs": True, "top_logprobs": 3})
    for tok in out["choices"][0]["logprobs"]["content"]:
        alts = ", ".join(f"{t['token']!r}: {t['logprob']:.2f}" for t in tok["top_logprobs"])
        print(f"{tok['token']!r:>12} {tok['logprob']:7.3f}   [{alts}]")


if __name__ == "__main__":
    main()
