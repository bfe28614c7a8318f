"""Function calling over the OpenAI-compatible server.

Start the server with a parser that matches the model's markup, e.g.

    python -m vllm_metax_b200.entrypoints.cli serve /path/to/Qwen3-8B --tool-call-parser hermes --reasoning-parser qwen3

then run this client.  It sends one question with a tool, executes the call the model asks for, sends the result back
and prints the final answer (plus the model's reasoning when a reasoning parser is set).
"""
import argparse
import json
import urllib.request


def post(url: str, body: dict) -> dict:
    req = urllib.request.Request(url, data=json.dumps(body).encode(), headers={"Content-Type": "application/json"})
    return json.loads(urllib.request.urlopen(req, timeout=600).read())


def get_weather(city: str) -> str:
    return json.dumps({"city": city, "forecast": "sunny", "high_c": 24})


TOOLS = [{"type": "function", "function": {
    "name": "get_weather", "description": "Weather forecast for a city",
    "parameters": {"type": "object", "properties": {"city": {"type": "string"}}, "required": ["city"]}}}]


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--url", default="http://127.0.0.1:8000/v1/chat/completions")
    ap.add_argument("--model", default="b200-model")
    ap.add_argument("--force", action="store_true", help="tool_choice names the function (constrained arguments)")
    a = ap.parse_args()
    messages = [{"role": "user", "content": "What is the weather in Paris today?"}]
    body = {"model": a.model, "messages": messages, "tools": TOOLS, "max_tokens": 512}
    if a.force:
        body["tool_choice"] = {"type": "function", "function": {"name": "get_weather"}}
    msg = post(a.url, body)["choices"][0]["message"]
    if msg.get("reasoning_content"):
        print("reasoning:", msg["reasoning_content"][:400])
    if not msg.get("tool_calls"):
        print("answer without a call:", msg.get("content"))
        return
    messages.append(msg)
    for call in msg["tool_calls"]:
        args = json.loads(call["function"]["arguments"])
        print("model calls", call["function"]["name"], args)
        messages.append({"role": "tool", "tool_call_id": call["id"], "content": get_weather(**args)})
    final = post(a.url, {"model": a.model, "messages": messages, "tools": TOOLS, "max_tokens": 256})
    print("answer:", final["choices"][0]["message"]["content"])


if __name__ == "__main__":
    main()
