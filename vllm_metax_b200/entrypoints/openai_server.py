"""OpenAI-compatible HTTP server over ``AsyncLLM``.

Routes: ``/v1/models``, ``/v1/completions``, ``/v1/chat/completions`` (streaming through server-sent
events), ``/tokenize``, ``/detokenize``, ``/health``, ``/metrics`` (Prometheus text), and the control
plane the RLHF / benchmark harnesses use: ``/sleep``, ``/wake_up``, ``/is_sleeping``, ``/pause``,
``/resume``, ``/collective_rpc``-free by design (SPMD ranks run the same server code).
Parity: the reference is served by ``vllm serve`` (OpenAI API server + ``vllm bench serve`` client,
tools/batched_test/bench_sweep.sh:3-14); sampling defaults follow patch/enhancement/chores/bench_serve_args.py:284-292
(temperature 0 unless the request sets one).
"""
import asyncio
import json
import time
import uuid

import torch
from typing import Any, Optional

from ..engine.llm import EngineDeadError
from ..engine.sampling_params import SamplingParams
from .async_engine import AsyncLLM


def sampling_from_request(body: dict, default_max_tokens: int = 16) -> SamplingParams:
    stop = body.get("stop")
    if isinstance(stop, str):
        stop = [stop]
    kw: dict[str, Any] = dict(
        max_tokens=int(body.get("max_tokens") or body.get("max_completion_tokens") or default_max_tokens),
        temperature=float(body.get("temperature", 0.0) or 0.0),
        top_p=float(body.get("top_p", 1.0) or 1.0),
        top_k=int(body.get("top_k", 0) or 0),
        min_p=float(body.get("min_p", 0.0) or 0.0),
        repetition_penalty=float(body.get("repetition_penalty", 1.0) or 1.0),
        presence_penalty=float(body.get("presence_penalty", 0.0) or 0.0),
        frequency_penalty=float(body.get("frequency_penalty", 0.0) or 0.0),
        ignore_eos=bool(body.get("ignore_eos", False)),
        seed=body.get("seed"),
    )
    lp = body.get("logprobs")
    if lp is True or (isinstance(lp, int) and not isinstance(lp, bool) and lp >= 0 and lp is not False):
        # chat: ``logprobs: true`` + ``top_logprobs: n``; completions: ``logprobs: n``
        kw["logprobs"] = int(body.get("top_logprobs") or 0) if lp is True else int(lp)
    if stop:
        kw["stop"] = list(stop)
    if body.get("include_stop_str_in_output"):
        kw["include_stop_str_in_output"] = True
    if body.get("bad_words"):
        kw["bad_words"] = list(body["bad_words"])
    if body.get("min_tokens"):
        kw["min_tokens"] = int(body["min_tokens"])
    if body.get("skip_special_tokens") is False:
        kw["skip_special_tokens"] = False
    if body.get("truncate_prompt_tokens"):
        kw["truncate_prompt_tokens"] = int(body["truncate_prompt_tokens"])
    if body.get("stop_token_ids"):
        kw["stop_token_ids"] = list(body["stop_token_ids"])
    so = body.get("structured_outputs") or {}
    choice = body.get("guided_choice") or so.get("choice")
    if choice:
        kw["guided_choice"] = list(choice)
    for name in ("guided_regex", "guided_json", "guided_grammar"):
        if body.get(name) is not None or so.get(name[7:]) is not None:
            kw[name] = body.get(name) if body.get(name) is not None else so.get(name[7:])
    rf = body.get("response_format")
    if isinstance(rf, dict) and not any(k in kw for k in ("guided_json", "guided_regex", "guided_choice", "guided_grammar")):
        kind = rf.get("type")
        if kind == "json_object":                 # any JSON object
            kw["guided_json"] = {"type": "object"}
        elif kind == "json_schema":               # {"type": "json_schema", "json_schema": {"name": ..., "schema": {...}}}
            js = rf.get("json_schema") or {}
            schema = js.get("schema", js.get("json_schema"))
            if not isinstance(schema, (dict, str)):
                raise ValueError("response_format.json_schema needs a 'schema' object")
            kw["guided_json"] = schema
        elif kind not in (None, "text"):
            raise ValueError(f"response_format type {kind!r} is not served (text, json_object, json_schema)")
    if body.get("allowed_token_ids"):
        kw["allowed_token_ids"] = [int(t) for t in body["allowed_token_ids"]]
    if body.get("logit_bias"):
        kw["logit_bias"] = {int(k): float(v) for k, v in body["logit_bias"].items()}
    fields = getattr(SamplingParams, "__dataclass_fields__", None)
    if fields is not None:
        kw = {k: v for k, v in kw.items() if k in fields}
    sp = SamplingParams(**kw)
    if body.get("priority"):
        sp._priority = int(body["priority"])        # scheduling policy "priority": smaller is served first
    return sp


def load_chat_template(arg: Optional[str]) -> Optional[str]:
    """``--chat-template``: a file with a Jinja template, or the template text itself."""
    if not arg:
        return None
    import os

    if os.path.exists(arg):
        with open(arg) as f:
            return f.read()
    if "{{" in arg or "{%" in arg:
        return arg
    raise ValueError(f"chat template {arg!r} is neither a file nor template text")


_TEMPLATE_CACHE: dict = {}


def _compile_template(text: str):
    """Jinja in a sandbox, with the conventions chat templates rely on (``raise_exception``, ``tojson``,
    whitespace control as in the tokenizers' own renderer)."""
    t = _TEMPLATE_CACHE.get(text)
    if t is None:
        from jinja2.sandbox import ImmutableSandboxedEnvironment

        def raise_exception(msg):
            raise ValueError(f"chat template: {msg}")

        env = ImmutableSandboxedEnvironment(trim_blocks=True, lstrip_blocks=True)
        env.globals["raise_exception"] = raise_exception
        env.filters["tojson"] = lambda x, **kw: json.dumps(x, ensure_ascii=False, **{k: v for k, v in kw.items() if k == "indent"})
        t = _TEMPLATE_CACHE[text] = env.from_string(text)
    return t


def render_chat(tokenizer, messages: list[dict], add_generation_prompt: bool = True, tools: Optional[list] = None,
                chat_template: Optional[str] = None, continue_final_message: bool = False,
                template_kwargs: Optional[dict] = None) -> str:
    """``continue_final_message``: the last message is an unfinished assistant turn; the prompt ends inside it (the
    template's end-of-turn text after that message is cut) and no generation prompt is added.  ``template_kwargs``
    are extra variables for the template (``enable_thinking`` and the like)."""
    if continue_final_message:
        if add_generation_prompt and messages and messages[-1].get("role") == "assistant":
            add_generation_prompt = False
        if add_generation_prompt:
            raise ValueError("continue_final_message and add_generation_prompt exclude each other")
        if not messages or not isinstance(messages[-1].get("content"), str):
            raise ValueError("continue_final_message needs a final message with text content")
        full = render_chat(tokenizer, messages, False, tools, chat_template, False, template_kwargs)
        tail = messages[-1]["content"].rstrip()
        at = full.rfind(tail)
        if at < 0:
            raise ValueError("the chat template does not reproduce the final message's text; cannot continue it")
        return full[: at + len(tail)]
    extra = {k: v for k, v in (template_kwargs or {}).items()
             if k not in ("messages", "tools", "add_generation_prompt", "bos_token", "eos_token", "tokenize")}
    if chat_template:        # the server's own template wins over the tokenizer's
        return _compile_template(chat_template).render(
            **extra, messages=messages, tools=tools or None, add_generation_prompt=add_generation_prompt,
            bos_token=getattr(tokenizer, "bos_token", None) or "", eos_token=getattr(tokenizer, "eos_token", None) or "")
    if tokenizer is not None and getattr(tokenizer, "chat_template", None):
        kw = {"tools": tools} if tools else {}
        return tokenizer.apply_chat_template(messages, tokenize=False, add_generation_prompt=add_generation_prompt,
                                             **kw, **extra)
    if tools:      # no template: list the functions in a system turn, Hermes style
        listing = "\n".join(json.dumps(t.get("function", t)) for t in tools)
        messages = [{"role": "system", "content": "You may call these functions by answering "
                     "<tool_call>{\"name\": ..., \"arguments\": {...}}</tool_call>:\n" + listing}] + list(messages)
    text = "".join(f"<|{m.get('role', 'user')}|>\n{m.get('content', '')}\n" for m in messages)
    return text + ("<|assistant|>\n" if add_generation_prompt else "")


def prometheus_text(allm: AsyncLLM) -> str:
    m, st = allm.metrics, allm.engine.stats
    kv = allm.engine.kv
    lines = []

    def g(name, val, typ="gauge", help_=""):
        lines.append(f"# HELP b200:{name} {help_}")
        lines.append(f"# TYPE b200:{name} {typ}")
        lines.append(f"b200:{name} {val}")

    g("num_requests_running", len(allm.engine.scheduler.running), help_="requests in the running queue")
    g("num_requests_waiting", len(allm.engine.scheduler.waiting), help_="requests waiting for admission")
    g("request_success_total", m["requests_finished"], "counter", "finished requests")
    g("request_aborted_total", m["requests_aborted"], "counter", "aborted requests")
    g("prompt_tokens_total", m["prompt_tokens"], "counter", "prompt tokens received")
    g("generation_tokens_total", m["generated_tokens"], "counter", "tokens generated")
    g("engine_steps_total", st["steps"], "counter", "scheduler iterations")
    g("num_preemptions_total", st["preemptions"], "counter", "preempted requests")
    g("time_to_first_token_seconds_sum", m["ttft_sum"], "counter", "sum of TTFT")
    g("time_to_first_token_seconds_count", m["ttft_count"], "counter", "TTFT samples")
    usage = getattr(kv, "usage", None)
    if callable(usage):
        g("kv_cache_usage_perc", usage(), help_="fraction of KV blocks in use")
    for h in getattr(allm, "histograms", {}).values():
        lines.append(h.render())
    return "\n".join(lines) + "\n"


def format_logprobs(entries: Optional[list], tokenizer, chat: bool, start: int = 0):
    """``request.logprobs`` entries -> the OpenAI ``logprobs`` object of a choice (chat or completions flavour)."""
    if entries is None:
        return None

    def name(tid: int) -> str:
        if tokenizer is None:
            return f"token_id:{tid}"
        return tokenizer.decode([tid])

    if chat:
        content = []
        for e in entries[start:]:
            tok = name(e["token_id"])
            content.append({"token": tok, "logprob": e["logprob"], "bytes": list(tok.encode("utf-8", "replace")),
                            "top_logprobs": [{"token": name(t), "logprob": v, "bytes": list(name(t).encode("utf-8", "replace"))}
                                             for t, v in e["top"]]})
        return {"content": content}
    toks = [name(e["token_id"]) for e in entries[start:]]
    offsets, o = [], 0
    for t in toks:
        offsets.append(o)
        o += len(t)
    return {"tokens": toks, "token_logprobs": [e["logprob"] for e in entries[start:]],
            "top_logprobs": [{name(t): v for t, v in e["top"]} for e in entries[start:]], "text_offset": offsets}


def build_app(allm: AsyncLLM, served_model_name: str = "b200-model", lora_modules: Optional[dict] = None,
              tool_call_parser: Optional[str] = None, reasoning_parser: Optional[str] = None,
              chat_template: Optional[str] = None):
    """``lora_modules``: adapter name -> ``LoRARequest``; a request whose ``model`` field names one runs with it.
    ``tool_call_parser`` / ``reasoning_parser``: names from ``entrypoints/parsers.py``; with them chat answers carry
    ``message.tool_calls`` / ``message.reasoning_content``."""
    from .parsers import get_reasoning_parser, get_tool_parser, parse_chat_output

    lora_modules = dict(lora_modules or {})
    chat_template = load_chat_template(chat_template)       # file or text; None: the tokenizer's own template
    tool_parser, think_parser = get_tool_parser(tool_call_parser), get_reasoning_parser(reasoning_parser)
    from fastapi import FastAPI, Request
    from fastapi.responses import JSONResponse, PlainTextResponse, StreamingResponse

    app = FastAPI(title="vllm_metax_b200 OpenAI-compatible server")
    tok = allm.engine.tokenizer
    llm = allm.llm
    state = {"sleeping": False}

    def encode(prompt) -> tuple[list[int], Optional[str]]:
        if isinstance(prompt, list) and prompt and isinstance(prompt[0], int):
            return list(prompt), None
        if isinstance(prompt, list) and len(prompt) == 1:
            prompt = prompt[0]
            if isinstance(prompt, list):
                return list(prompt), None
        if not isinstance(prompt, str):
            raise ValueError("prompt must be a string or a list of token ids")
        if tok is None:
            raise ValueError("text prompt given but the server has no tokenizer; send token ids")
        return tok.encode(prompt), prompt

    IMAGE_MARK = "<|b200-image|>"

    def split_images(messages: list) -> tuple[list, list]:
        """OpenAI content parts -> (messages with plain-text content where every image is ``IMAGE_MARK``, PIL images).
        Images come as ``data:`` URLs (base64); remote URLs are refused - the server fetches nothing."""
        import base64
        import io

        images, flat = [], []
        for m in messages:
            c = m.get("content")
            if not isinstance(c, list):
                flat.append(m)
                continue
            text = ""
            for part in c:
                kind = part.get("type")
                if kind == "text":
                    text += part.get("text", "")
                elif kind == "image_url":
                    url = (part.get("image_url") or {}).get("url", "")
                    if not url.startswith("data:") or "," not in url:
                        raise ValueError("image_url must be a data: URL (base64); remote images are not fetched")
                    from PIL import Image

                    images.append(Image.open(io.BytesIO(base64.b64decode(url.split(",", 1)[1]))).convert("RGB"))
                    text += IMAGE_MARK
                else:
                    raise ValueError(f"unsupported content part type {kind!r}")
            flat.append(dict(m, content=text))
        return flat, images

    def encode_with_images(text: str, n_images: int) -> list[int]:
        """Tokenise around the image marks and put the model's placeholder id where each image goes."""
        model = llm.engine.runner.model
        if not getattr(model, "is_multimodal", False):
            raise ValueError("this model takes no image inputs")
        pieces = text.split(IMAGE_MARK)
        if len(pieces) != n_images + 1:
            raise ValueError("image marks were altered by the chat template")
        ids = list(tok.encode(pieces[0]))
        for piece in pieces[1:]:
            ids.append(model.image_token_id)
            if piece:
                try:
                    ids.extend(tok.encode(piece, add_special_tokens=False))
                except TypeError:
                    ids.extend(tok.encode(piece))
        return ids

    def err(status: int, msg: str, typ: str = "invalid_request_error"):
        return JSONResponse({"error": {"message": msg, "type": typ, "code": status}}, status_code=status)

    @app.get("/health")
    async def health():
        return PlainTextResponse("", status_code=503 if allm.is_dead else 200)

    @app.get("/v1/models")
    async def models():
        base = {"id": served_model_name, "object": "model", "owned_by": "b200",
                "max_model_len": llm.engine.cfg.scheduler.max_model_len}
        adapters = [{"id": n, "object": "model", "owned_by": "b200", "parent": served_model_name} for n in lora_modules]
        return {"object": "list", "data": [base] + adapters}

    @app.get("/metrics")
    async def metrics():
        return PlainTextResponse(prometheus_text(allm))

    @app.post("/tokenize")
    async def tokenize(req: Request):
        body = await req.json()
        if tok is None:
            return err(400, "no tokenizer")
        ids = tok.encode(body.get("prompt", ""))
        return {"tokens": ids, "count": len(ids), "max_model_len": llm.engine.cfg.scheduler.max_model_len}

    @app.post("/detokenize")
    async def detokenize(req: Request):
        body = await req.json()
        if tok is None:
            return err(400, "no tokenizer")
        return {"prompt": tok.decode(body.get("tokens", []))}

    @app.post("/sleep")
    async def sleep(level: int = 1):
        llm.sleep(level)
        state["sleeping"] = True
        return {"status": "sleeping", "level": level}

    @app.post("/wake_up")
    async def wake_up(req: Request):
        tags = req.query_params.getlist("tags") or None
        llm.wake_up(tags)
        state["sleeping"] = False
        return {"status": "awake"}

    @app.get("/is_sleeping")
    async def is_sleeping():
        return {"is_sleeping": state["sleeping"]}

    @app.post("/pause")
    async def pause():
        llm.pause_generation()
        return {"status": "paused"}

    @app.post("/resume")
    async def resume():
        llm.resume_generation()
        return {"status": "running"}

    async def run_one(ids, prompt, params, rid, traceparent=None):
        last = None
        async for chunk in allm.generate(ids, params, rid, prompt, traceparent):
            last = chunk
        return last

    def usage(prompt_tokens: int, completion_tokens: int) -> dict:
        return {"prompt_tokens": prompt_tokens, "completion_tokens": completion_tokens,
                "total_tokens": prompt_tokens + completion_tokens}

    async def serve(body: dict, chat: bool, traceparent: Optional[str] = None):
        try:
            images = []
            tools = body.get("tools") if chat else None
            tool_choice = body.get("tool_choice", "auto" if tools else "none")
            forced_tool = None
            if tools and tool_choice == "none":
                tools = None
            if tools and isinstance(tool_choice, dict):          # {"type": "function", "function": {"name": ...}}
                forced_tool = (tool_choice.get("function") or {}).get("name")
                spec = next((t.get("function", t) for t in tools if t.get("function", t).get("name") == forced_tool), None)
                if spec is None:
                    return err(400, f"tool_choice names an unknown function {forced_tool!r}")
                body = dict(body, guided_json=spec.get("parameters") or {"type": "object"})   # the answer IS the arguments
            if tools and tool_choice == "required":              # at least one call: the answer is a JSON list of calls
                one = [{"type": "object", "required": ["name", "parameters"],
                        "properties": {"name": {"const": t.get("function", t).get("name")},
                                       "parameters": t.get("function", t).get("parameters") or {"type": "object"}}}
                       for t in tools]
                forced_tool = True
                body = dict(body, guided_json={"type": "array", "minItems": 1, "items": {"anyOf": one}})
            if tools and tool_parser is None and forced_tool is None and tool_choice != "auto":
                return err(400, "tool_choice needs the server to be started with --tool-call-parser")
            if chat:
                messages, images = split_images(body.get("messages") or [])
                text = render_chat(tok, messages, tools=tools,
                                   add_generation_prompt=bool(body.get("add_generation_prompt", True)),
                                   chat_template=body.get("chat_template") or chat_template,
                                   continue_final_message=bool(body.get("continue_final_message", False)),
                                   template_kwargs=body.get("chat_template_kwargs"))
                if images:
                    ids, prompt = encode_with_images(text, len(images)), text
                else:
                    ids, prompt = encode(text)
            else:
                ids, prompt = encode(body.get("prompt", ""))
            params = sampling_from_request(body, default_max_tokens=16 if not chat else 256)
            if images:
                params._multi_modal_data = {"image": images}
            model_name = body.get("model")
            if model_name in lora_modules:
                params._lora_request = lora_modules[model_name]
            elif model_name not in (None, "", served_model_name):
                return err(404, f"model {model_name!r} is not served (adapters: {sorted(lora_modules)})", "model_not_found")
        except Exception as e:
            return err(400, str(e))
        if len(ids) + params.max_tokens > llm.engine.cfg.scheduler.max_model_len:
            return err(400, f"prompt ({len(ids)}) + max_tokens ({params.max_tokens}) exceeds max_model_len")
        rid = ("chatcmpl-" if chat else "cmpl-") + uuid.uuid4().hex[:16]
        created = int(time.time())
        obj = "chat.completion" if chat else "text_completion"
        n_samples = max(1, int(body.get("n") or 1))
        if n_samples > 1 and body.get("stream"):
            return err(400, "n > 1 is served for non-streaming requests only")
        if int(body.get("best_of") or 0) > n_samples:
            return err(400, "best_of > n is served by the offline API (SamplingParams.best_of), not by this server")

        def sample_params(i: int):
            if n_samples == 1:
                return params
            import copy

            p_i = copy.copy(params)                     # independent samples; a seeded request stays reproducible
            p_i.seed = None if params.seed is None else params.seed + i
            for extra in ("_multi_modal_data", "_lora_request"):
                if hasattr(params, extra):
                    setattr(p_i, extra, getattr(params, extra))
            return p_i

        def build_choice(i: int, last) -> dict:
            text = last.text if last.text is not None else ""
            if chat:
                msg = parse_chat_output(text, tool_parser, think_parser, bool(tools), forced_tool)
                message = {"role": "assistant", "content": msg.content}
                if msg.reasoning_content is not None:
                    message["reasoning_content"] = msg.reasoning_content
                finish = last.finish_reason
                if msg.tool_calls:
                    message["tool_calls"] = [c.to_openai() for c in msg.tool_calls]
                    finish = "tool_calls" if forced_tool in (None, True) else finish
                return {"index": i, "message": message, "finish_reason": finish,
                        "logprobs": format_logprobs(last.logprobs, tok, True)}
            return {"index": i, "text": text, "token_ids": last.token_ids,
                    "logprobs": format_logprobs(last.logprobs, tok, False), "finish_reason": last.finish_reason}

        if not body.get("stream"):
            try:
                lasts = await asyncio.gather(*[
                    run_one(ids, prompt, sample_params(i), rid if n_samples == 1 else f"{rid}-{i}", traceparent)
                    for i in range(n_samples)])
            except EngineDeadError as e:
                return err(500, str(e), "engine_dead")
            return {"id": rid, "object": obj, "created": created, "model": served_model_name,
                    "choices": [build_choice(i, last) for i, last in enumerate(lasts)],
                    "usage": usage(len(ids), sum(len(last.token_ids) for last in lasts))}

        # with a tool or reasoning parser the markup has to be complete before it can be split, so such a stream
        # carries the parsed message in its last chunk; plain chats stream token by token
        parse_at_end = chat and (forced_tool is not None or think_parser is not None
                                 or (tool_parser is not None and bool(tools)))

        async def sse():
            prev = ""
            ntok = 0
            sent_lp = 0
            try:
                async for chunk in allm.generate(ids, params, rid, prompt, traceparent):
                    cur = chunk.text if chunk.text is not None else ""
                    delta, prev = cur[len(prev):] if cur.startswith(prev) else cur, cur
                    ntok = len(chunk.token_ids)
                    lp = format_logprobs(chunk.logprobs, tok, chat, sent_lp)
                    sent_lp = len(chunk.logprobs) if chunk.logprobs is not None else 0
                    if parse_at_end:
                        if not chunk.finished:
                            continue
                        msg = parse_chat_output(cur, tool_parser, think_parser, bool(tools), forced_tool)
                        d = {"role": "assistant", "content": msg.content}
                        if msg.reasoning_content is not None:
                            d["reasoning_content"] = msg.reasoning_content
                        finish = chunk.finish_reason
                        if msg.tool_calls:
                            d["tool_calls"] = [c.to_openai(i) for i, c in enumerate(msg.tool_calls)]
                            finish = "tool_calls" if forced_tool in (None, True) else finish
                        ch = {"index": 0, "delta": d, "finish_reason": finish,
                              "logprobs": format_logprobs(chunk.logprobs, tok, True)}
                    elif chat:
                        ch = {"index": 0, "delta": {"content": delta}, "finish_reason": chunk.finish_reason, "logprobs": lp}
                    else:
                        ch = {"index": 0, "text": delta, "token_ids": chunk.new_token_ids, "logprobs": lp,
                              "finish_reason": chunk.finish_reason}
                    yield "data: " + json.dumps({"id": rid, "object": obj + (".chunk" if chat else ""), "created": created,
                                                 "model": served_model_name, "choices": [ch]}) + "\n\n"
                if (body.get("stream_options") or {}).get("include_usage"):
                    yield "data: " + json.dumps({"id": rid, "object": obj, "created": created, "model": served_model_name,
                                                 "choices": [], "usage": usage(len(ids), ntok)}) + "\n\n"
            except EngineDeadError as e:
                yield "data: " + json.dumps({"error": {"message": str(e), "type": "engine_dead", "code": 500}}) + "\n\n"
            yield "data: [DONE]\n\n"

        return StreamingResponse(sse(), media_type="text/event-stream")

    # ---- Responses API (non-streaming subset): the chat path under another envelope
    @app.post("/v1/responses")
    async def responses(req: Request):
        """``input``: a string or a list of ``{"role", "content"}`` items (content a string or a list of
        ``input_text`` / ``output_text`` parts); ``instructions`` becomes the system turn.  Answers one ``message``
        output item (plus a ``reasoning`` item and ``function_call`` items when the parsers find them)."""
        body = await req.json()
        if body.get("stream"):
            return err(400, "the responses route is served without streaming; use /v1/chat/completions to stream")
        inp = body.get("input", "")
        messages = []
        if body.get("instructions"):
            messages.append({"role": "system", "content": str(body["instructions"])})
        if isinstance(inp, str):
            messages.append({"role": "user", "content": inp})
        else:
            for item in inp:
                c = item.get("content", "")
                if isinstance(c, list):
                    c = "".join(p.get("text", "") for p in c if p.get("type") in ("input_text", "output_text", "text"))
                messages.append({"role": item.get("role", "user"), "content": c})
        chat_body = {k: v for k, v in body.items() if k in ("temperature", "top_p", "seed", "model", "stop", "top_k")}
        chat_body.update(messages=messages, max_tokens=body.get("max_output_tokens") or 256)
        tools = [t for t in (body.get("tools") or []) if t.get("type") == "function"]
        if tools:       # Responses puts name / parameters at the top level of a tool
            chat_body["tools"] = [{"type": "function", "function": {k: t[k] for k in ("name", "description", "parameters")
                                                                  if k in t}} for t in tools]
            if body.get("tool_choice") in ("auto", "none"):
                chat_body["tool_choice"] = body["tool_choice"]
        out = await serve(chat_body, chat=True, traceparent=req.headers.get("traceparent"))
        if not isinstance(out, dict):
            return out                                       # an error response
        msg = out["choices"][0]["message"]
        items = []
        if msg.get("reasoning_content"):
            items.append({"type": "reasoning", "id": "rs_" + uuid.uuid4().hex[:16],
                          "summary": [{"type": "summary_text", "text": msg["reasoning_content"]}]})
        for c in msg.get("tool_calls") or []:
            items.append({"type": "function_call", "id": "fc_" + uuid.uuid4().hex[:16], "call_id": c["id"],
                          "name": c["function"]["name"], "arguments": c["function"]["arguments"], "status": "completed"})
        if msg.get("content") is not None or not items:
            items.append({"type": "message", "id": "msg_" + uuid.uuid4().hex[:16], "role": "assistant", "status": "completed",
                          "content": [{"type": "output_text", "text": msg.get("content") or "", "annotations": []}]})
        u = out["usage"]
        finish = out["choices"][0]["finish_reason"]
        return {"id": "resp_" + uuid.uuid4().hex[:16], "object": "response", "created_at": out["created"],
                "model": out["model"], "status": "completed" if finish != "length" else "incomplete",
                "incomplete_details": {"reason": "max_output_tokens"} if finish == "length" else None,
                "output": items, "output_text": msg.get("content") or "",
                "usage": {"input_tokens": u["prompt_tokens"], "output_tokens": u["completion_tokens"],
                          "total_tokens": u["total_tokens"]}}

    # ---- pooling endpoints: embeddings, similarity scores, re-ranking (they drive the engine from its own thread)
    def many(x) -> list:
        """``str | [int] -> [x]``; ``[str] | [[int]]`` stay lists."""
        if isinstance(x, str) or (isinstance(x, list) and x and isinstance(x[0], int)):
            return [x]
        if not isinstance(x, list) or not x:
            raise ValueError("input must be a string, a list of strings, or token ids")
        return list(x)

    def count_tokens(items: list) -> int:
        return sum(len(encode(i)[0]) for i in items)

    @app.post("/v1/embeddings")
    async def embeddings(req: Request):
        body = await req.json()
        try:
            items = many(body.get("input"))
            ntok = count_tokens(items)
            pooling = body.get("pooling", "last")
            normalize = bool(body.get("normalize", True))
            emb = await allm.call(lambda: llm.embed(items, pooling=pooling, normalize=normalize))
        except EngineDeadError as e:
            return err(500, str(e), "engine_dead")
        except Exception as e:  # noqa: BLE001
            return err(400, str(e))
        dims = body.get("dimensions")
        if dims:                                   # matryoshka-style truncation + renormalisation
            emb = torch.nn.functional.normalize(emb[:, : int(dims)], dim=-1) if normalize else emb[:, : int(dims)]
        if body.get("encoding_format") == "base64":
            import base64

            import numpy as np

            data = [base64.b64encode(np.asarray(e, dtype=np.float32).tobytes()).decode() for e in emb.tolist()]
        else:
            data = emb.tolist()
        return {"id": "embd-" + uuid.uuid4().hex[:16], "object": "list", "model": served_model_name,
                "data": [{"object": "embedding", "index": i, "embedding": e} for i, e in enumerate(data)],
                "usage": {"prompt_tokens": ntok, "total_tokens": ntok}}

    @app.post("/pooling")
    async def pooling_route(req: Request):
        """The pooled hidden state of every input, not normalised unless asked; ``task``: ``embed`` (default; one
        vector per input) or ``token_embed`` is not served."""
        body = await req.json()
        if body.get("task", "embed") not in ("embed", "encode"):
            return err(400, f"pooling task {body.get('task')!r} is not served (embed)")
        try:
            items = many(body.get("input"))
            ntok = count_tokens(items)
            emb = await allm.call(lambda: llm.embed(items, pooling=body.get("pooling", "last"),
                                                    normalize=bool(body.get("normalize", False))))
        except EngineDeadError as e:
            return err(500, str(e), "engine_dead")
        except Exception as e:  # noqa: BLE001
            return err(400, str(e))
        return {"id": "pool-" + uuid.uuid4().hex[:16], "object": "list", "model": served_model_name,
                "data": [{"object": "pooling", "index": i, "data": e} for i, e in enumerate(emb.tolist())],
                "usage": {"prompt_tokens": ntok, "total_tokens": ntok}}

    async def score_impl(body: dict):
        t1 = body.get("text_1", body.get("query"))
        t2 = body.get("text_2", body.get("documents"))
        if t1 is None or t2 is None:
            raise ValueError("text_1 and text_2 (or query and documents) are required")
        one = isinstance(t1, str) or (isinstance(t1, list) and t1 and isinstance(t1[0], int))
        docs = many(t2)
        scores = await allm.call(lambda: llm.score(t1 if one else list(t1), docs))
        return docs, [float(x) for x in scores], count_tokens(docs) + count_tokens([t1] if one else list(t1))

    @app.post("/score")
    @app.post("/v1/score")
    async def score(req: Request):
        try:
            docs, scores, ntok = await score_impl(await req.json())
        except EngineDeadError as e:
            return err(500, str(e), "engine_dead")
        except Exception as e:  # noqa: BLE001
            return err(400, str(e))
        return {"id": "score-" + uuid.uuid4().hex[:16], "object": "list", "model": served_model_name,
                "data": [{"index": i, "object": "score", "score": x} for i, x in enumerate(scores)],
                "usage": {"prompt_tokens": ntok, "total_tokens": ntok}}

    @app.post("/rerank")
    @app.post("/v1/rerank")
    @app.post("/v2/rerank")
    async def rerank(req: Request):
        body = await req.json()
        try:
            docs, scores, ntok = await score_impl(body)
        except EngineDeadError as e:
            return err(500, str(e), "engine_dead")
        except Exception as e:  # noqa: BLE001
            return err(400, str(e))
        order = sorted(range(len(docs)), key=lambda i: -scores[i])[: int(body.get("top_n") or len(docs))]
        return {"id": "rerank-" + uuid.uuid4().hex[:16], "model": served_model_name,
                "usage": {"total_tokens": ntok},
                "results": [{"index": i, "document": {"text": docs[i] if isinstance(docs[i], str) else None},
                             "relevance_score": scores[i]} for i in order]}

    @app.post("/classify")
    async def classify(req: Request):
        """``class_token_ids``: the token whose logit stands for each class (label-token classification); answers the
        softmax over them for every input."""
        body = await req.json()
        try:
            items = many(body.get("input"))
            ids = [int(t) for t in body.get("class_token_ids") or []]
            if len(ids) < 2:
                raise ValueError("class_token_ids needs at least two token ids")
            probs = await allm.call(lambda: llm.classify(items, ids))
        except EngineDeadError as e:
            return err(500, str(e), "engine_dead")
        except Exception as e:  # noqa: BLE001
            return err(400, str(e))
        return {"id": "classify-" + uuid.uuid4().hex[:16], "object": "list", "model": served_model_name,
                "data": [{"index": i, "label": int(torch.as_tensor(p).argmax()), "probs": [float(x) for x in p],
                          "num_classes": len(ids)} for i, p in enumerate(probs.tolist())]}

    # ---- administration -------------------------------------------------------------------------------------------
    @app.get("/version")
    async def version():
        from ..version import __version__

        return {"version": __version__}

    @app.get("/server_info")
    async def server_info():
        """The engine's resolved configuration (what upstream's development endpoint of this name answers)."""
        import dataclasses

        def plain(v):
            if dataclasses.is_dataclass(v) and not isinstance(v, type):
                return {f.name: plain(getattr(v, f.name)) for f in dataclasses.fields(v)}
            if isinstance(v, (list, tuple)):
                return [plain(x) for x in v]
            if isinstance(v, dict):
                return {str(k): plain(x) for k, x in v.items()}
            return v if isinstance(v, (int, float, str, bool, type(None))) else str(v)

        cfg = llm.engine.cfg
        out = {name: plain(getattr(cfg, name)) for name in ("parallel", "scheduler", "cache") if hasattr(cfg, name)}
        m = getattr(cfg, "model", None)
        if m is not None:
            out["model"] = {k: plain(getattr(m, k)) for k in ("architecture", "dtype", "num_hidden_layers", "hidden_size",
                                                                "num_attention_heads", "num_key_value_heads", "vocab_size",
                                                                "max_position_embeddings") if hasattr(m, k)}
        from ..version import __version__

        return {"version": __version__, "served_model_name": served_model_name, "config": out}

    @app.get("/ping")
    @app.post("/ping")
    async def ping():
        if llm.engine.dead is not None:
            return err(500, str(llm.engine.dead), "engine_dead")
        return {}

    @app.post("/reset_prefix_cache")
    async def reset_prefix_cache():
        n = await allm.call(lambda: llm.engine.kv.reset_prefix_cache())
        return {"status": "ok", "blocks_dropped": int(n or 0)}

    @app.post("/v1/load_lora_adapter")
    async def load_lora_adapter(req: Request):
        body = await req.json()
        name, path = body.get("lora_name"), body.get("lora_path")
        if not name or not path:
            return err(400, "lora_name and lora_path are required")
        if getattr(llm.engine.runner, "lora", None) is None:
            return err(400, "the server was started without --enable-lora")
        from ..lora import LoRARequest

        next_id = 1 + max([getattr(r, "lora_int_id", 0) for r in lora_modules.values()] + [0])
        lora_modules[name] = LoRARequest(name, next_id, path)
        return {"status": "ok", "lora_name": name}

    @app.post("/v1/unload_lora_adapter")
    async def unload_lora_adapter(req: Request):
        name = (await req.json()).get("lora_name")
        if name not in lora_modules:
            return err(404, f"adapter {name!r} is not loaded", "model_not_found")
        del lora_modules[name]
        return {"status": "ok", "lora_name": name}

    async def serve_batch(body: dict, traceparent: Optional[str] = None):
        """``/v1/completions`` with several prompts and / or ``echo`` (non-streaming): choice ``i * n + j`` is sample j
        of prompt i.  ``echo`` puts the prompt in front of the text and, with ``logprobs``, the log-probability of every
        prompt token in front of the completion's (first token: null) - what evaluation harnesses use to score a
        continuation; ``max_tokens: 0`` then generates nothing."""
        try:
            raw = body.get("prompt", "")
            single = isinstance(raw, str) or (isinstance(raw, list) and raw and isinstance(raw[0], int))
            items = [raw] if single else list(raw)
            if not items:
                raise ValueError("prompt is empty")
            enc = [encode(p) for p in items]
            echo = bool(body.get("echo"))
            no_gen = body.get("max_tokens") == 0
            if no_gen and not echo:
                raise ValueError("max_tokens = 0 needs echo")
            params = sampling_from_request(dict(body, max_tokens=1) if no_gen else body, default_max_tokens=16)
            model_name = body.get("model")
            if model_name in lora_modules:
                params._lora_request = lora_modules[model_name]
            elif model_name not in (None, "", served_model_name):
                return err(404, f"model {model_name!r} is not served (adapters: {sorted(lora_modules)})", "model_not_found")
            limit = llm.engine.cfg.scheduler.max_model_len
            for ids, _ in enc:
                if len(ids) + params.max_tokens > limit:
                    raise ValueError(f"prompt ({len(ids)}) + max_tokens ({params.max_tokens}) exceeds max_model_len")
        except Exception as e:  # noqa: BLE001
            return err(400, str(e))
        n_samples = max(1, int(body.get("n") or 1))
        rid = "cmpl-" + uuid.uuid4().hex[:16]
        import copy

        def p_for(j: int):
            p_j = copy.copy(params)
            if n_samples > 1:
                p_j.seed = None if params.seed is None else params.seed + j
            if hasattr(params, "_lora_request"):
                p_j._lora_request = params._lora_request
            return p_j

        try:
            lasts = await asyncio.gather(*[run_one(ids, text, p_for(j), f"{rid}-{i}-{j}", traceparent)
                                           for i, (ids, text) in enumerate(enc) for j in range(n_samples)])
            plp = None
            if echo and params.logprobs is not None:
                k = int(params.logprobs)
                plp = await allm.call(lambda: llm.prompt_logprobs([ids for ids, _ in enc], top=k))
        except EngineDeadError as e:
            return err(500, str(e), "engine_dead")
        choices, completion_tokens = [], 0
        for i, (ids, text) in enumerate(enc):
            ptext = text if text is not None else (tok.decode(ids) if tok is not None else "")
            for j in range(n_samples):
                last = lasts[i * n_samples + j]
                gen_text = "" if no_gen else (last.text or "")
                gen_ids = [] if no_gen else last.token_ids
                gen_lp = [] if no_gen else (last.logprobs or [])
                completion_tokens += len(gen_ids)
                lp_obj = None
                if params.logprobs is not None:
                    entries = (plp[i] if plp is not None else []) + list(gen_lp)
                    real = [e for e in entries if e is not None]
                    lp_obj = format_logprobs(real, tok, False)
                    if plp is not None and lp_obj is not None:           # the first prompt token has no prediction
                        first = tok.decode([ids[0]]) if tok is not None else f"token_id:{ids[0]}"
                        lp_obj = {"tokens": [first] + lp_obj["tokens"], "token_logprobs": [None] + lp_obj["token_logprobs"],
                                  "top_logprobs": [None] + lp_obj["top_logprobs"],
                                  "text_offset": [0] + [o + len(first) for o in lp_obj["text_offset"]]}
                choices.append({"index": i * n_samples + j, "text": (ptext if echo else "") + gen_text,
                                "token_ids": gen_ids, "logprobs": lp_obj,
                                "finish_reason": "length" if no_gen else last.finish_reason})
        return {"id": rid, "object": "text_completion", "created": int(time.time()), "model": served_model_name,
                "choices": choices, "usage": usage(sum(len(ids) for ids, _ in enc), completion_tokens)}

    @app.post("/v1/completions")
    async def completions(req: Request):
        body = await req.json()
        raw = body.get("prompt")
        several = isinstance(raw, list) and len(raw) > 1 and not isinstance(raw[0], int)
        if several or body.get("echo"):
            if body.get("stream"):
                return err(400, "several prompts / echo are served for non-streaming requests only")
            return await serve_batch(body, req.headers.get("traceparent"))
        return await serve(body, chat=False, traceparent=req.headers.get("traceparent"))

    @app.post("/v1/chat/completions")
    async def chat_completions(req: Request):
        return await serve(await req.json(), chat=True, traceparent=req.headers.get("traceparent"))

    return app
