"""OpenAI-compatible server over a tiny random model on CPU (in-process ASGI client, no sockets)."""
import asyncio
import json
import os

import pytest
import torch

from vllm_metax_b200 import LLM, ModelConfig
from vllm_metax_b200.entrypoints.async_engine import AsyncLLM
from vllm_metax_b200.entrypoints.openai_server import build_app, sampling_from_request


class ToyTokenizer:
    chat_template = None

    def encode(self, text):
        return [3 + (ord(c) % 200) for c in text][:64] or [3]

    def decode(self, ids, skip_special_tokens=True):
        return "".join(chr(97 + (i % 26)) for i in ids)


@pytest.fixture(scope="module")
def client_app():
    cfg = ModelConfig(architecture="LlamaForCausalLM", vocab_size=256, hidden_size=64, intermediate_size=128,
                      num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2, head_dim=16,
                      max_position_embeddings=256, dtype=torch.float32)
    llm = LLM(cfg, device="cpu", load_format="dummy", num_gpu_blocks=64, block_size=16, max_model_len=256,
              tokenizer=ToyTokenizer(), seed=0)
    allm = AsyncLLM(llm)
    yield allm, build_app(allm, "toy")
    allm.shutdown()


def _call(app, method, path, body=None):
    import httpx

    async def go():
        transport = httpx.ASGITransport(app=app)
        async with httpx.AsyncClient(transport=transport, base_url="http://test") as c:
            r = await c.request(method, path, json=body)
            return r.status_code, r.text
    return asyncio.run(go())


def test_sampling_defaults_are_greedy():
    sp = sampling_from_request({"max_tokens": 5})
    assert sp.temperature == 0.0 and sp.max_tokens == 5


def test_models_health_metrics(client_app):
    allm, app = client_app
    pytest.importorskip("httpx")
    assert _call(app, "GET", "/health")[0] == 200
    code, text = _call(app, "GET", "/v1/models")
    assert code == 200 and json.loads(text)["data"][0]["id"] == "toy"
    code, text = _call(app, "GET", "/metrics")
    assert code == 200 and "b200:generation_tokens_total" in text


def test_completion_and_chat(client_app):
    allm, app = client_app
    pytest.importorskip("httpx")
    code, text = _call(app, "POST", "/v1/completions", {"prompt": "hello", "max_tokens": 6, "ignore_eos": True})
    out = json.loads(text)
    assert code == 200 and out["usage"]["completion_tokens"] == 6 and len(out["choices"][0]["text"]) == 6
    # token-id prompt, identical result on repeat (greedy)
    code, text2 = _call(app, "POST", "/v1/completions", {"prompt": "hello", "max_tokens": 6, "ignore_eos": True})
    assert json.loads(text2)["choices"][0]["text"] == out["choices"][0]["text"]
    code, text = _call(app, "POST", "/v1/chat/completions",
                       {"messages": [{"role": "user", "content": "hi"}], "max_tokens": 4, "ignore_eos": True})
    assert code == 200 and json.loads(text)["choices"][0]["message"]["role"] == "assistant"


def test_streaming(client_app):
    allm, app = client_app
    pytest.importorskip("httpx")
    code, text = _call(app, "POST", "/v1/completions", {"prompt": [5, 6, 7], "max_tokens": 5, "stream": True,
                                                         "ignore_eos": True, "stream_options": {"include_usage": True}})
    assert code == 200
    events = [json.loads(l[6:]) for l in text.splitlines() if l.startswith("data: ") and l != "data: [DONE]"]
    toks = [t for e in events if e["choices"] for t in e["choices"][0]["token_ids"]]
    assert len(toks) == 5 and events[-1]["usage"]["completion_tokens"] == 5
    assert text.rstrip().endswith("data: [DONE]")


def test_too_long_prompt_is_rejected(client_app):
    allm, app = client_app
    pytest.importorskip("httpx")
    code, text = _call(app, "POST", "/v1/completions", {"prompt": [1] * 250, "max_tokens": 50})
    assert code == 400 and "max_model_len" in text


def test_constrained_and_unknown_model(client_app):
    allm, app = client_app
    pytest.importorskip("httpx")
    body = {"prompt": "pick", "max_tokens": 8, "guided_choice": [[10, 11], [12]], "model": "toy"}
    code, text = _call(app, "POST", "/v1/completions", body)
    out = json.loads(text)
    assert code == 200 and out["choices"][0]["token_ids"] in ([10, 11], [12]) and out["choices"][0]["finish_reason"] == "stop"
    body = {"prompt": "pick", "max_tokens": 5, "ignore_eos": True, "allowed_token_ids": [7, 8]}
    code, text = _call(app, "POST", "/v1/completions", body)
    assert code == 200 and set(json.loads(text)["choices"][0]["token_ids"]) <= {7, 8}
    code, text = _call(app, "POST", "/v1/completions", {"prompt": "x", "guided_regex": "[a-c]{4}", "max_tokens": 12})
    assert code == 200 and len(json.loads(text)["choices"][0]["text"]) == 4
    code, text = _call(app, "POST", "/v1/completions", {"prompt": "x", "model": "no-such-adapter"})
    assert code == 404 and "not served" in text


def test_lora_adapter_selected_by_model_name():
    pytest.importorskip("httpx")
    from vllm_metax_b200.lora import LoRARequest

    cfg = ModelConfig(architecture="LlamaForCausalLM", vocab_size=256, hidden_size=64, intermediate_size=128,
                      num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2, head_dim=16,
                      max_position_embeddings=256, dtype=torch.float32)
    llm = LLM(cfg, device="cpu", load_format="dummy", num_gpu_blocks=64, block_size=16, max_model_len=256,
              tokenizer=ToyTokenizer(), seed=0, enable_lora=True, max_loras=2, max_lora_rank=4)
    g = torch.Generator().manual_seed(0)
    t = {}
    for i in range(2):
        stem = f"base_model.model.model.layers.{i}.self_attn.q_proj"
        t[stem + ".lora_A.weight"] = torch.randn(4, 64, generator=g)
        t[stem + ".lora_B.weight"] = torch.randn(64, 4, generator=g)
    allm = AsyncLLM(llm)
    try:
        app = build_app(allm, "toy", {"tuned": LoRARequest("tuned", 1, tensors=t, config={"lora_alpha": 8})})
        code, text = _call(app, "GET", "/v1/models")
        assert [m["id"] for m in json.loads(text)["data"]] == ["toy", "tuned"]
        req = {"prompt": "hello there", "max_tokens": 8, "ignore_eos": True}
        base = json.loads(_call(app, "POST", "/v1/completions", dict(req, model="toy"))[1])["choices"][0]["token_ids"]
        tuned = json.loads(_call(app, "POST", "/v1/completions", dict(req, model="tuned"))[1])["choices"][0]["token_ids"]
        assert len(tuned) == 8 and tuned != base
        assert llm.engine.runner.lora.list_adapters() == [1]
    finally:
        allm.shutdown()


def test_tracing_and_latency_histograms():
    """One span per finished request reaches an OTLP/HTTP collector (a fake one here), continuing the caller's
    trace; /metrics exposes the latency histograms."""
    pytest.importorskip("httpx")
    import http.server
    import threading

    from vllm_metax_b200.utils.observability import Histogram, RequestTracer, parse_traceparent

    got = []

    class Collector(http.server.BaseHTTPRequestHandler):
        def do_POST(self):
            got.append((self.path, json.loads(self.rfile.read(int(self.headers["Content-Length"])))))
            self.send_response(200)
            self.end_headers()

        def log_message(self, *a):
            pass

    srv = http.server.HTTPServer(("127.0.0.1", 0), Collector)
    threading.Thread(target=srv.serve_forever, daemon=True).start()
    cfg = ModelConfig(architecture="LlamaForCausalLM", vocab_size=256, hidden_size=64, intermediate_size=128,
                      num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2, head_dim=16,
                      max_position_embeddings=256, dtype=torch.float32)
    llm = LLM(cfg, device="cpu", load_format="dummy", num_gpu_blocks=64, block_size=16, max_model_len=256,
              tokenizer=ToyTokenizer(), seed=0)
    tracer = RequestTracer.from_endpoint(f"http://127.0.0.1:{srv.server_port}", "toy")
    allm = AsyncLLM(llm, tracer)
    try:
        app = build_app(allm, "toy")

        async def go():
            import httpx

            async with httpx.AsyncClient(transport=httpx.ASGITransport(app=app), base_url="http://test") as c:
                tp = "00-0af7651916cd43dd8448eb211c80319c-b7ad6b7169203331-01"
                r = await c.post("/v1/completions", json={"prompt": "hello", "max_tokens": 5, "ignore_eos": True},
                                 headers={"traceparent": tp})
                m = await c.get("/metrics")
                return r.status_code, m.text

        code, metrics = asyncio.run(go())
        assert code == 200
        tracer.exporter.flush()
        assert got and got[0][0] == "/v1/traces"
        span = got[0][1]["resourceSpans"][0]["scopeSpans"][0]["spans"][0]
        assert span["traceId"] == "0af7651916cd43dd8448eb211c80319c" and span["parentSpanId"] == "b7ad6b7169203331"
        attrs = {a["key"]: a["value"] for a in span["attributes"]}
        assert attrs["gen_ai.usage.completion_tokens"]["intValue"] == "5"
        assert "gen_ai.latency.time_to_first_token" in attrs and "gen_ai.latency.e2e" in attrs
        assert 'b200:time_to_first_token_seconds_bucket{le="+Inf"} 1' in metrics
        assert "b200:inter_token_latency_seconds_count 4" in metrics and "b200:e2e_request_latency_seconds_sum" in metrics
    finally:
        allm.shutdown()
        srv.shutdown()
    assert parse_traceparent("garbage") == (None, None)
    h = Histogram("x", "h", (1.0, 2.0))
    for v in (0.5, 1.5, 3.0):
        h.observe(v)
    assert 'x_bucket{le="2.0"} 2' in h.render("") and 'x_bucket{le="+Inf"} 3' in h.render("")


def test_logprobs_in_completions_and_chat(client_app):
    allm, app = client_app
    pytest.importorskip("httpx")
    code, text = _call(app, "POST", "/v1/completions", {"model": "toy", "prompt": "hello", "max_tokens": 4, "logprobs": 2})
    assert code == 200, text
    lp = json.loads(text)["choices"][0]["logprobs"]
    assert len(lp["tokens"]) == 4 and len(lp["token_logprobs"]) == 4 and all(len(t) <= 2 for t in lp["top_logprobs"])
    assert all(v <= 0.0 for v in lp["token_logprobs"])
    code, text = _call(app, "POST", "/v1/chat/completions", {"model": "toy", "messages": [{"role": "user", "content": "hi"}],
                                                             "max_tokens": 3, "logprobs": True, "top_logprobs": 3})
    assert code == 200, text
    content = json.loads(text)["choices"][0]["logprobs"]["content"]
    assert len(content) == 3 and all(len(c["top_logprobs"]) == 3 for c in content)
    # greedy decoding: the sampled token is the most likely one
    assert all(c["logprob"] == max(t["logprob"] for t in c["top_logprobs"]) for c in content)
    code, text = _call(app, "POST", "/v1/completions", {"model": "toy", "prompt": "hello", "max_tokens": 2})
    assert json.loads(text)["choices"][0]["logprobs"] is None


def test_chat_with_tools_and_reasoning_parsers():
    """A server started with parsers: a request with ``tools`` is rendered with the function list and answered with the
    parsed message (the toy model writes no markup, so the answer stays content); ``tool_choice`` needs a parser."""
    pytest.importorskip("httpx")
    cfg = ModelConfig(architecture="LlamaForCausalLM", vocab_size=256, hidden_size=64, intermediate_size=128,
                      num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2, head_dim=16,
                      max_position_embeddings=256, dtype=torch.float32)
    llm = LLM(cfg, device="cpu", load_format="dummy", num_gpu_blocks=64, block_size=16, max_model_len=256,
              tokenizer=ToyTokenizer(), seed=0)
    allm = AsyncLLM(llm)
    try:
        app = build_app(allm, "toy", tool_call_parser="hermes", reasoning_parser="deepseek_r1")
        tools = [{"type": "function", "function": {"name": "get_weather", "parameters": {"type": "object", "properties": {}}}}]
        body = {"model": "toy", "messages": [{"role": "user", "content": "weather?"}], "max_tokens": 4, "tools": tools}
        code, text = _call(app, "POST", "/v1/chat/completions", body)
        assert code == 200, text
        msg = json.loads(text)["choices"][0]["message"]
        assert msg["role"] == "assistant" and "tool_calls" not in msg and msg["content"]
        code, text = _call(app, "POST", "/v1/chat/completions", dict(body, stream=True))
        assert code == 200 and text.count("data: ") == 2 and "[DONE]" in text     # one parsed chunk + the terminator
        plain = build_app(allm, "toy")
        code, text = _call(plain, "POST", "/v1/chat/completions", dict(body, tool_choice={"type": "function", "function": {"name": "nope"}}))
        assert code == 400 and "unknown function" in text
    finally:
        allm.shutdown()


def test_pooling_and_admin_endpoints(client_app):
    """Embeddings / score / rerank / classify run on the engine thread while the server keeps generating; the
    answers equal the offline API."""
    pytest.importorskip("httpx")
    allm, app = client_app
    llm = allm.llm
    texts = ["hello world", "another sentence here", "hello world"]
    code, text = _call(app, "POST", "/v1/embeddings", {"input": texts})
    res = json.loads(text)
    assert code == 200 and [d["index"] for d in res["data"]] == [0, 1, 2]
    emb = torch.tensor([d["embedding"] for d in res["data"]])
    assert emb.shape == (3, 64) and torch.allclose(emb.norm(dim=-1), torch.ones(3), atol=1e-4)
    assert torch.allclose(emb[0], emb[2], atol=1e-5) and not torch.allclose(emb[0], emb[1], atol=1e-3)
    assert res["usage"]["prompt_tokens"] == sum(len(llm.tokenizer.encode(t)) for t in texts)
    code, text = _call(app, "POST", "/v1/embeddings", {"input": "hello world", "dimensions": 16, "encoding_format": "base64"})
    import base64

    import numpy as np
    small = np.frombuffer(base64.b64decode(json.loads(text)["data"][0]["embedding"]), dtype=np.float32)
    assert small.shape == (16,) and abs(float(np.linalg.norm(small)) - 1.0) < 1e-4
    code, text = _call(app, "POST", "/score", {"text_1": "hello world", "text_2": ["hello world", "zzz qqq"]})
    sc = [d["score"] for d in json.loads(text)["data"]]
    assert code == 200 and abs(sc[0] - 1.0) < 1e-4 and sc[1] < sc[0]
    code, text = _call(app, "POST", "/v1/rerank", {"query": "hello world", "documents": ["zzz qqq", "hello world", "abc"],
                                                   "top_n": 2})
    rr = json.loads(text)["results"]
    assert code == 200 and len(rr) == 2 and rr[0]["index"] == 1 and rr[0]["document"]["text"] == "hello world"
    assert rr[0]["relevance_score"] >= rr[1]["relevance_score"]
    code, text = _call(app, "POST", "/classify", {"input": ["good", "bad"], "class_token_ids": [5, 9, 11]})
    cl = json.loads(text)["data"]
    assert code == 200 and len(cl) == 2 and abs(sum(cl[0]["probs"]) - 1.0) < 1e-4 and cl[0]["num_classes"] == 3
    assert _call(app, "POST", "/classify", {"input": "x", "class_token_ids": [1]})[0] == 400
    assert _call(app, "POST", "/v1/embeddings", {"input": []})[0] == 400
    assert json.loads(_call(app, "GET", "/version")[1])["version"]
    assert _call(app, "GET", "/ping")[0] == 200
    assert _call(app, "POST", "/reset_prefix_cache")[0] == 200
    assert _call(app, "POST", "/v1/load_lora_adapter", {"lora_name": "a", "lora_path": "/x"})[0] == 400   # no --enable-lora
    assert _call(app, "POST", "/v1/unload_lora_adapter", {"lora_name": "nope"})[0] == 404


def test_embeddings_while_generating(client_app):
    """A generation request that is in flight when an embedding call takes the engine still finishes with the same
    tokens."""
    pytest.importorskip("httpx")
    import httpx

    allm, app = client_app
    body = {"prompt": "the quick brown fox", "max_tokens": 40}
    want = json.loads(_call(app, "POST", "/v1/completions", body)[1])["choices"][0]["token_ids"]

    async def go():
        transport = httpx.ASGITransport(app=app)
        async with httpx.AsyncClient(transport=transport, base_url="http://test") as c:
            gen = asyncio.create_task(c.post("/v1/completions", json=body))
            await asyncio.sleep(0.02)
            embs = await asyncio.gather(*[c.post("/v1/embeddings", json={"input": ["abc def", "ghi"]}) for _ in range(3)])
            return await gen, embs
    gen, embs = asyncio.run(go())
    assert gen.status_code == 200 and json.loads(gen.text)["choices"][0]["token_ids"] == want
    assert all(e.status_code == 200 and len(json.loads(e.text)["data"]) == 2 for e in embs)


def test_chat_templates():
    """The shipped Jinja templates render conversations (with tools, tool calls and tool results), and a server
    started with one uses it instead of the tokenizer's."""
    from vllm_metax_b200.entrypoints.openai_server import load_chat_template, render_chat

    root = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "examples", "chat_templates")
    msgs = [{"role": "system", "content": "be brief"}, {"role": "user", "content": "weather in Paris?"}]
    chatml = load_chat_template(os.path.join(root, "chatml.jinja"))
    text = render_chat(None, msgs, chat_template=chatml)
    assert text == "<|im_start|>system\nbe brief<|im_end|>\n<|im_start|>user\nweather in Paris?<|im_end|>\n<|im_start|>assistant\n"
    assert render_chat(None, msgs, add_generation_prompt=False, chat_template=chatml).endswith("Paris?<|im_end|>\n")
    tools = [{"type": "function", "function": {"name": "get_weather", "parameters": {"type": "object",
                                                                                   "properties": {"city": {"type": "string"}}}}}]
    convo = msgs + [{"role": "assistant", "content": "", "tool_calls": [
        {"type": "function", "function": {"name": "get_weather", "arguments": {"city": "Paris"}}}]},
        {"role": "tool", "content": "18 C"}]
    hermes = render_chat(None, convo, tools=tools, chat_template=load_chat_template(os.path.join(root, "hermes_tools.jinja")))
    assert '"name": "get_weather"' in hermes and "<tools>" in hermes and "<tool_response>\n18 C\n</tool_response>" in hermes
    assert '<tool_call>\n{"name": "get_weather", "arguments": {"city": "Paris"}}\n</tool_call>' in hermes
    from vllm_metax_b200.entrypoints.parsers import parse_hermes
    call = parse_hermes(hermes[hermes.index("<|im_start|>assistant"):hermes.index("<|im_start|>user\n<tool_response>")]).tool_calls[0]
    assert call.name == "get_weather" and json.loads(call.arguments) == {"city": "Paris"}      # what it renders, the parser reads
    llama = render_chat(type("T", (), {"bos_token": "<|begin_of_text|>", "eos_token": ""})(), convo, tools=tools,
                        chat_template=load_chat_template(os.path.join(root, "llama3_json_tools.jinja")))
    assert llama.startswith("<|begin_of_text|><|start_header_id|>system<|end_header_id|>")
    assert '{"name": "get_weather", "parameters": {"city": "Paris"}}<|eot_id|>' in llama
    assert llama.endswith("<|start_header_id|>assistant<|end_header_id|>\n\n")
    with pytest.raises(ValueError):
        load_chat_template("no-such-file")
    inline = load_chat_template("{% for m in messages %}[{{ m['role'] }}]{{ m['content'] }}{% endfor %}")
    assert render_chat(None, msgs, chat_template=inline) == "[system]be brief[user]weather in Paris?"


def test_server_uses_its_chat_template(client_app):
    pytest.importorskip("httpx")
    allm, _ = client_app
    seen = {}
    tok = allm.engine.tokenizer
    orig = tok.encode

    def spy(text, *a, **kw):
        seen["text"] = text
        return orig(text)
    tok.encode = spy
    try:
        app = build_app(allm, "toy", chat_template="{% for m in messages %}<{{ m['role'] }}>{{ m['content'] }}{% endfor %}<bot>")
        code, _ = _call(app, "POST", "/v1/chat/completions", {"messages": [{"role": "user", "content": "hi"}], "max_tokens": 3})
        assert code == 200 and seen["text"] == "<user>hi<bot>"
        code, _ = _call(app, "POST", "/v1/chat/completions", {"messages": [{"role": "user", "content": "hi"}], "max_tokens": 3,
                                                              "chat_template": "{{ messages[0]['content'] }}!"})
        assert code == 200 and seen["text"] == "hi!"
    finally:
        tok.encode = orig


def test_completions_with_several_prompts_and_echo(client_app):
    """Batch prompts give one choice per (prompt, sample); ``echo`` + ``logprobs`` + ``max_tokens: 0`` scores the
    prompt itself - the way evaluation harnesses ask for the log-likelihood of a continuation."""
    pytest.importorskip("httpx")
    allm, app = client_app
    llm = allm.llm
    code, text = _call(app, "POST", "/v1/completions", {"prompt": ["hello", "bye now"], "max_tokens": 4, "n": 2,
                                                        "temperature": 1.0, "seed": 5})
    res = json.loads(text)
    assert code == 200 and [c["index"] for c in res["choices"]] == [0, 1, 2, 3]
    one = json.loads(_call(app, "POST", "/v1/completions", {"prompt": "bye now", "max_tokens": 4, "n": 2,
                                                            "temperature": 1.0, "seed": 5})[1])
    assert [c["token_ids"] for c in res["choices"][2:]] == [c["token_ids"] for c in one["choices"]]
    assert res["usage"]["completion_tokens"] == 16
    # scoring: prompt log-probabilities through the server equal the offline API
    prompt = "the quick brown fox"
    ids = llm.tokenizer.encode(prompt)
    want = llm.prompt_logprobs([ids], top=2)[0]
    code, text = _call(app, "POST", "/v1/completions", {"prompt": prompt, "max_tokens": 0, "echo": True, "logprobs": 2})
    ch = json.loads(text)["choices"][0]
    assert code == 200 and ch["text"] == prompt and ch["token_ids"] == []
    lp = ch["logprobs"]
    assert lp["token_logprobs"][0] is None and len(lp["token_logprobs"]) == len(ids)
    assert all(abs(a - b["logprob"]) < 1e-5 for a, b in zip(lp["token_logprobs"][1:], want[1:]))
    assert lp["top_logprobs"][0] is None and len(lp["top_logprobs"][1]) == 2
    assert lp["text_offset"][:3] == [0, 1, 2]
    # echo with a continuation: prompt text in front, prompt + completion log-probabilities
    code, text = _call(app, "POST", "/v1/completions", {"prompt": prompt, "max_tokens": 3, "echo": True, "logprobs": 1})
    ch = json.loads(text)["choices"][0]
    assert ch["text"].startswith(prompt) and len(ch["text"]) == len(prompt) + 3
    assert len(ch["logprobs"]["token_logprobs"]) == len(ids) + 3
    assert _call(app, "POST", "/v1/completions", {"prompt": ["a", "b"], "stream": True})[0] == 400
    assert _call(app, "POST", "/v1/completions", {"prompt": "a", "max_tokens": 0})[0] in (200, 400)


def test_responses_route(client_app):
    pytest.importorskip("httpx")
    allm, app = client_app
    code, text = _call(app, "POST", "/v1/responses", {"input": "hi there", "instructions": "be brief", "max_output_tokens": 5})
    res = json.loads(text)
    assert code == 200 and res["object"] == "response" and res["status"] == "incomplete"
    msg = [o for o in res["output"] if o["type"] == "message"][0]
    assert msg["content"][0]["type"] == "output_text" and msg["content"][0]["text"] == res["output_text"]
    assert res["usage"]["output_tokens"] == 5 and res["usage"]["input_tokens"] > 0
    chat = json.loads(_call(app, "POST", "/v1/chat/completions", {"messages": [
        {"role": "system", "content": "be brief"}, {"role": "user", "content": "hi there"}], "max_tokens": 5})[1])
    assert chat["choices"][0]["message"]["content"] == res["output_text"]          # the same request underneath
    code, text = _call(app, "POST", "/v1/responses", {"input": [
        {"role": "user", "content": [{"type": "input_text", "text": "hi "}, {"type": "input_text", "text": "there"}]}],
        "instructions": "be brief", "max_output_tokens": 5})
    assert json.loads(text)["output_text"] == res["output_text"]
    assert _call(app, "POST", "/v1/responses", {"input": "x", "stream": True})[0] == 400


def test_response_format_and_chat_rendering_options(client_app):
    """``response_format`` maps onto JSON-guided decoding; ``continue_final_message``, ``add_generation_prompt`` and
    ``chat_template_kwargs`` reach the template; ``/pooling`` and ``/server_info`` answer."""
    from vllm_metax_b200.entrypoints.openai_server import load_chat_template, render_chat

    schema = {"type": "object", "properties": {"a": {"type": "integer"}}, "required": ["a"]}
    assert sampling_from_request({"response_format": {"type": "json_object"}}).guided_json == {"type": "object"}
    assert sampling_from_request({"response_format": {"type": "json_schema",
                                                      "json_schema": {"name": "x", "schema": schema}}}).guided_json == schema
    assert sampling_from_request({"response_format": {"type": "text"}}).guided_json is None
    assert sampling_from_request({"guided_regex": "a+", "response_format": {"type": "json_object"}}).guided_json is None
    with pytest.raises(ValueError):
        sampling_from_request({"response_format": {"type": "structural_tag"}})
    assert sampling_from_request({"guided_grammar": 'root ::= "a"+'}).guided_grammar == 'root ::= "a"+'
    assert sampling_from_request({"structured_outputs": {"grammar": 'root ::= "b"'}}).guided_grammar == 'root ::= "b"'

    root = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "examples", "chat_templates")
    chatml = load_chat_template(os.path.join(root, "chatml.jinja"))
    msgs = [{"role": "user", "content": "count"}, {"role": "assistant", "content": "one, two,"}]
    text = render_chat(None, msgs, chat_template=chatml, continue_final_message=True)
    assert text == "<|im_start|>user\ncount<|im_end|>\n<|im_start|>assistant\none, two,"          # the turn stays open
    with pytest.raises(ValueError):
        render_chat(None, msgs[:1], chat_template=chatml, continue_final_message=True)          # a user turn cannot be continued
    think = "{{ messages[0]['content'] }}{% if enable_thinking %}<think>{% endif %}"
    assert render_chat(None, msgs, chat_template=think, template_kwargs={"enable_thinking": True}) == "count<think>"
    assert render_chat(None, msgs, chat_template=think, template_kwargs={"enable_thinking": False}) == "count"

    pytest.importorskip("httpx")
    allm, app = client_app
    seen = {}
    tok = allm.engine.tokenizer
    orig = tok.encode

    def spy(text, *a, **kw):
        seen["text"] = text
        return orig(text)
    tok.encode = spy
    try:
        code, _ = _call(app, "POST", "/v1/chat/completions", {"messages": msgs, "max_tokens": 3, "chat_template": chatml,
                                                              "continue_final_message": True, "add_generation_prompt": False})
        assert code == 200 and seen["text"].endswith("<|im_start|>assistant\none, two,")
        code, _ = _call(app, "POST", "/v1/chat/completions", {"messages": msgs[:1], "max_tokens": 3, "chat_template": think,
                                                              "chat_template_kwargs": {"enable_thinking": True}})
        assert code == 200 and seen["text"] == "count<think>"
        code, _ = _call(app, "POST", "/v1/chat/completions", {"messages": msgs[:1], "max_tokens": 3, "chat_template": chatml,
                                                              "add_generation_prompt": False})
        assert code == 200 and seen["text"].endswith("count<|im_end|>\n")
        code, text = _call(app, "POST", "/v1/chat/completions", {"messages": msgs[:1], "max_tokens": 3,
                                                                 "response_format": {"type": "nope"}})
        assert code == 400 and "response_format" in text
    finally:
        tok.encode = orig
    code, text = _call(app, "POST", "/pooling", {"input": ["hello", "wor"]})
    out = json.loads(text)
    assert code == 200 and [d["object"] for d in out["data"]] == ["pooling", "pooling"] and len(out["data"][0]["data"]) == 64
    code, emb = _call(app, "POST", "/v1/embeddings", {"input": ["hello"], "normalize": False})
    torch.testing.assert_close(torch.tensor(out["data"][0]["data"]), torch.tensor(json.loads(emb)["data"][0]["embedding"]))
    assert _call(app, "POST", "/pooling", {"input": "x", "task": "token_classify"})[0] == 400
    code, text = _call(app, "GET", "/server_info")
    info = json.loads(text)
    assert code == 200 and info["served_model_name"] == "toy" and info["config"]["scheduler"]["max_model_len"] == 256


def test_tool_choice_required_and_named_are_served_by_guided_json():
    """``tool_choice="required"`` constrains the answer to a JSON list of calls of the offered functions, a named
    function to its arguments; neither needs a tool-call parser.  (Character-level tokenizer: the random model can
    spell JSON.)"""
    pytest.importorskip("httpx")
    from tests.test_structured import CHARS
    from tests.test_structured import CharTokenizer as _Chars

    class CharTokenizer(_Chars):
        def encode(self, text, add_special_tokens=True):           # the chat rendering has newlines
            return [CHARS.index(c) if c in CHARS else 0 for c in text][-200:]

    cfg = ModelConfig(architecture="LlamaForCausalLM", vocab_size=256, hidden_size=64, intermediate_size=128,
                      num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2, head_dim=16,
                      max_position_embeddings=512, dtype=torch.float32)
    llm = LLM(cfg, device="cpu", load_format="dummy", num_gpu_blocks=96, block_size=16, max_model_len=512,
              tokenizer=CharTokenizer(), seed=0)
    allm = AsyncLLM(llm)
    try:
        app = build_app(allm, "toy")
        tools = [{"type": "function", "function": {"name": "get_weather", "parameters": {
                      "type": "object", "properties": {"city": {"enum": ["Paris", "Rome"]}, "days": {"type": "integer", "minimum": 1, "maximum": 7}}}}},
                 {"type": "function", "function": {"name": "get_time", "parameters": {
                      "type": "object", "properties": {"zone": {"enum": ["UTC", "CET"]}}}}}]
        body = {"messages": [{"role": "user", "content": "weather?"}], "max_tokens": 200, "tools": tools,
                "temperature": 0.8, "seed": 2}
        code, text = _call(app, "POST", "/v1/chat/completions", dict(body, tool_choice="required"))
        assert code == 200, text
        choice = json.loads(text)["choices"][0]
        calls = choice["message"].get("tool_calls")
        if choice["finish_reason"] == "length":           # an unbounded list may outlast the limit: content, no calls
            assert not calls
        else:
            assert calls and choice["finish_reason"] == "tool_calls" and choice["message"]["content"] is None
            for c in calls:
                args = json.loads(c["function"]["arguments"])
                if c["function"]["name"] == "get_weather":
                    assert args["city"] in ("Paris", "Rome") and 1 <= args["days"] <= 7
                else:
                    assert c["function"]["name"] == "get_time" and args["zone"] in ("UTC", "CET")
        code, text = _call(app, "POST", "/v1/chat/completions",
                           dict(body, tool_choice={"type": "function", "function": {"name": "get_time"}}))
        assert code == 200, text
        call = json.loads(text)["choices"][0]["message"]["tool_calls"][0]["function"]
        assert call["name"] == "get_time" and json.loads(call["arguments"])["zone"] in ("UTC", "CET")
    finally:
        allm.shutdown()


def test_best_of_is_refused_by_the_server(client_app):
    pytest.importorskip("httpx")
    _, app = client_app
    code, text = _call(app, "POST", "/v1/completions", {"prompt": "hi", "max_tokens": 3, "n": 1, "best_of": 4})
    assert code == 400 and "best_of" in text
    assert _call(app, "POST", "/v1/completions", {"prompt": "hi", "max_tokens": 3, "n": 2, "best_of": 2})[0] == 200
