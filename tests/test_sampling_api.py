"""User-facing sampling parameters beyond the sampler itself: stop strings (with an incremental detokeniser that
survives multi-token characters), ``include_stop_str_in_output``, ``bad_words``, ``n`` samples per prompt,
``truncate_prompt_tokens`` - offline and through the OpenAI server."""
import asyncio
import json
import os
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

from tests.test_e2e_plumbing import tiny_cfg  # noqa: E402
from tests.test_structured import CharTokenizer  # noqa: E402

PRINTABLE = list(range(95))        # the character tokens of CharTokenizer


def _sp(**kw):
    """Seeded sampling over the printable tokens: varied text that a second run reproduces."""
    from vllm_metax_b200 import SamplingParams

    base = dict(max_tokens=30, temperature=1.0, seed=11, allowed_token_ids=PRINTABLE)
    base.update(kw)
    return SamplingParams(**base)


KW = dict(device="cpu", block_size=16, max_model_len=256, max_num_seqs=8, max_num_batched_tokens=64, num_gpu_blocks=64)


@pytest.fixture(scope="module")
def llm():
    from vllm_metax_b200 import LLM

    return LLM(tiny_cfg(), tokenizer=CharTokenizer(), **KW)


def test_stop_checker_waits_for_complete_characters():
    from vllm_metax_b200.engine.sampling_params import StopStringChecker

    class ByteTok:                      # one token per UTF-8 byte: a character is printable only when all bytes arrived
        def decode(self, ids, skip_special_tokens=True):
            return bytes(ids).decode("utf-8", errors="replace")

    text = "aé中 END tail"
    ids = list(text.encode("utf-8"))
    ck = StopStringChecker(ByteTok(), ["END"], include=False)
    hit_at = None
    for i in range(1, len(ids) + 1):
        if ck.step(ids[:i]) is not None:
            hit_at = i
            break
    assert hit_at == len("aé中 END".encode("utf-8"))
    assert ck.text == "aé中 " and "�" not in ck.text
    ck2 = StopStringChecker(ByteTok(), ["END", "中"], include=True)
    for i in range(1, len(ids) + 1):
        if ck2.step(ids[:i]) is not None:
            break
    assert ck2.hit == "中" and ck2.text == "aé中"      # the earliest stop wins, kept in the text


def test_stop_strings_end_generation_and_cut_the_text(llm):
    from vllm_metax_b200 import SamplingParams

    free = llm.generate(["Q: ok?"], _sp())[0].outputs[0]
    assert len(free.text) >= 12 and len(set(free.text)) > 4
    stop = free.text[6:9]                                   # a string the seeded continuation is known to contain
    cut = free.text.index(stop)
    got = llm.generate(["Q: ok?"], _sp(stop=[stop, "\x00never"]))[0].outputs[0]
    assert got.finish_reason == "stop" and got.stop_reason == stop
    assert got.text == free.text[:cut]
    assert len(got.token_ids) < len(free.token_ids)
    keep = llm.generate(["Q: ok?"], _sp(stop=[stop], include_stop_str_in_output=True))[0].outputs[0]
    assert keep.text == free.text[:cut + len(stop)]
    none = llm.generate(["Q: ok?"], _sp(stop=["\x00never"]))[0].outputs[0]
    assert none.text == free.text and none.finish_reason == "length" and none.stop_reason is None


def test_bad_words_never_appear(llm):
    from vllm_metax_b200 import SamplingParams

    free = llm.generate(["Q: ok?"], _sp(max_tokens=24))[0].outputs[0]
    first = free.token_ids[0]
    pair = free.token_ids[3:5]
    got = llm.generate(["Q: ok?"], _sp(max_tokens=24, bad_words=[[first], pair]))[0].outputs[0]
    assert first not in got.token_ids
    assert all(got.token_ids[i:i + 2] != pair for i in range(len(got.token_ids) - 1))
    word = free.text[2:4]
    got = llm.generate(["Q: ok?"], _sp(max_tokens=24, bad_words=[word]))[0].outputs[0]
    assert word not in got.text


def test_n_samples_per_prompt(llm):
    from vllm_metax_b200 import SamplingParams

    outs = llm.generate(["Q: ok?", "x"], SamplingParams(max_tokens=12, temperature=1.0, seed=7, n=3))
    assert len(outs) == 2 and all(len(o.outputs) == 3 for o in outs)
    assert [c.index for c in outs[0].outputs] == [0, 1, 2]
    assert len({tuple(c.token_ids) for c in outs[0].outputs}) > 1                  # independent samples
    again = llm.generate(["Q: ok?"], SamplingParams(max_tokens=12, temperature=1.0, seed=7, n=3))[0]
    assert [c.token_ids for c in again.outputs] == [c.token_ids for c in outs[0].outputs]     # seeded: reproducible
    greedy = llm.generate(["Q: ok?"], SamplingParams(max_tokens=6, n=2))[0]
    assert greedy.outputs[0].token_ids == greedy.outputs[1].token_ids


def test_truncate_prompt_tokens(llm):
    from vllm_metax_b200 import SamplingParams

    long = "abcdefghijklmnopqrstuvwxyz"
    a = llm.generate([long], SamplingParams(max_tokens=6, truncate_prompt_tokens=5))[0]
    b = llm.generate([long[-5:]], SamplingParams(max_tokens=6))[0]
    assert a.outputs[0].token_ids == b.outputs[0].token_ids and len(a.prompt_token_ids) == 5


def _call(app, body, path="/v1/completions"):
    import httpx

    async def go():
        transport = httpx.ASGITransport(app=app)
        async with httpx.AsyncClient(transport=transport, base_url="http://test") as c:
            r = await c.post(path, json=body)
            return r.status_code, r.text
    return asyncio.run(go())


def test_server_stop_and_n(llm):
    pytest.importorskip("httpx")
    from vllm_metax_b200.entrypoints.async_engine import AsyncLLM
    from vllm_metax_b200.entrypoints.openai_server import build_app, sampling_from_request

    sp = sampling_from_request({"stop": "ab", "include_stop_str_in_output": True, "bad_words": ["x"], "min_tokens": 2})
    assert sp.stop == ["ab"] and sp.include_stop_str_in_output and sp.bad_words == ["x"] and sp.min_tokens == 2
    allm = AsyncLLM(llm)
    try:
        app = build_app(allm, "toy")
        base = {"prompt": "Q: ok?", "max_tokens": 30, "temperature": 1.0, "seed": 11, "allowed_token_ids": PRINTABLE}
        code, text = _call(app, base)
        free = json.loads(text)["choices"][0]["text"]
        stop = free[6:9]
        code, text = _call(app, dict(base, stop=[stop]))
        ch = json.loads(text)["choices"][0]
        assert code == 200 and ch["text"] == free[:free.index(stop)] and ch["finish_reason"] == "stop"
        code, text = _call(app, {"prompt": "Q: ok?", "max_tokens": 8, "n": 3, "temperature": 1.0, "seed": 3})
        res = json.loads(text)
        assert code == 200 and [c["index"] for c in res["choices"]] == [0, 1, 2]
        assert res["usage"]["completion_tokens"] == 24
        code, text = _call(app, {"prompt": "Q: ok?", "max_tokens": 8, "n": 2, "stream": True})
        assert code == 400
        # a stream never shows the beginning of a stop string that then completes
        import httpx

        async def stream():
            transport = httpx.ASGITransport(app=app)
            async with httpx.AsyncClient(transport=transport, base_url="http://test") as c:
                async with c.stream("POST", "/v1/completions",
                                    json=dict(base, stop=[stop], stream=True)) as r:
                    parts = []
                    async for line in r.aiter_lines():
                        if line.startswith("data: ") and line != "data: [DONE]":
                            parts.append(json.loads(line[6:])["choices"][0]["text"])
                    return "".join(parts)
        assert asyncio.run(stream()) == free[:free.index(stop)]
    finally:
        allm.shutdown()


def test_beam_search_finds_a_more_likely_sequence_than_greedy(llm):
    """Against an exhaustive oracle on a short horizon: the best beam (width = all candidates that matter) has the
    highest total log-probability, and it is at least as likely as the greedy continuation."""
    from vllm_metax_b200 import SamplingParams

    prompt = "Q: ok?"
    beams = llm.beam_search([prompt], beam_width=4, max_tokens=3, ignore_eos=True)[0]
    assert len(beams) == 4 and all(len(b["token_ids"]) == 3 for b in beams)
    assert beams == sorted(beams, key=lambda b: -b["score"])
    greedy = llm.generate([prompt], SamplingParams(max_tokens=3, temperature=0.0, logprobs=1, ignore_eos=True))[0].outputs[0]
    g_lp = sum(e["logprob"] for e in greedy.logprobs)
    assert beams[0]["cum_logprob"] >= g_lp - 1e-4
    assert any(b["token_ids"] == greedy.token_ids for b in beams) or beams[-1]["cum_logprob"] > g_lp
    # the reported log-probability of the best beam is what the model assigns to it token by token
    ids = llm._to_ids(prompt)[0]
    total = 0.0
    for i, t in enumerate(beams[0]["token_ids"]):
        o = llm.generate([ids + beams[0]["token_ids"][:i]], SamplingParams(max_tokens=1, logprobs=8, ignore_eos=True))[0]
        top = dict(o.outputs[0].logprobs[0]["top"])
        total += top[t]
    assert abs(total - beams[0]["cum_logprob"]) < 1e-3


def test_prompt_logprobs_match_step_by_step_scoring(llm):
    """Chunked over several prefill steps (the prompt is longer than the step budget) and equal to what one decode
    step per prefix reports."""
    from vllm_metax_b200 import SamplingParams

    g = torch.Generator().manual_seed(2)
    ids = torch.randint(0, 95, (90,), generator=g).tolist()          # 90 tokens > the 64-token step budget
    got = llm.prompt_logprobs([ids, ids[:7]], top=3)
    assert got[0][0] is None and len(got[0]) == 90 and len(got[1]) == 7
    assert [e["token_id"] for e in got[0][1:]] == ids[1:]
    for k in (1, 5, 63, 64, 65, 89):                                  # around the chunk boundary too
        o = llm.generate([ids[:k]], SamplingParams(max_tokens=1, logprobs=1024, ignore_eos=True))[0]
        want = dict(o.outputs[0].logprobs[0]["top"])[ids[k]]
        assert abs(got[0][k]["logprob"] - want) < 1e-4, (k, got[0][k], want)
        assert len(got[0][k]["top"]) == 3 and got[0][k]["top"][0][1] >= got[0][k]["logprob"] - 1e-6
    assert abs(got[1][3]["logprob"] - got[0][3]["logprob"]) < 1e-4


def test_incremental_detokenizer_equals_full_decode():
    """A byte-level BPE tokenizer with a small vocabulary (multi-byte characters are split over several tokens):
    feeding the tokens a few at a time gives exactly the text of one full decode, never shows a broken character,
    and the final flush emits a trailing incomplete one the way the full decode does."""
    import random

    tokenizers = pytest.importorskip("tokenizers")
    from tokenizers import Tokenizer, decoders, models, pre_tokenizers, trainers

    from vllm_metax_b200.engine.sampling_params import IncrementalDetokenizer

    tok = Tokenizer(models.BPE(unk_token=None))
    tok.pre_tokenizer = pre_tokenizers.ByteLevel(add_prefix_space=False)
    tok.decoder = decoders.ByteLevel()
    corpus = ["the quick brown fox jumps over the lazy dog ", "héllo wörld çà et là ", "中文 测试 文本 ", "emoji 😀 🎉 ok "] * 5
    tok.train_from_iterator(corpus, trainers.BpeTrainer(vocab_size=300, initial_alphabet=pre_tokenizers.ByteLevel.alphabet(),
                                                        show_progress=False))

    class Wrap:                                  # the decode signature the engine uses
        def decode(self, ids, skip_special_tokens=True):
            return tok.decode(list(ids), skip_special_tokens=skip_special_tokens)

    rng = random.Random(0)
    pieces = ["the lazy dog", " héllo", " 中文测试", " 😀🎉", " wörld", " fox", "文本", " çà"]
    for trial in range(20):
        text = "".join(rng.choice(pieces) for _ in range(12))
        ids = tok.encode(text).ids
        assert len(ids) > len(text) // 3                       # the vocabulary really splits characters
        d = IncrementalDetokenizer(Wrap())
        i, seen = 0, ""
        while i < len(ids):
            i = min(len(ids), i + rng.randint(1, 3))
            d.step(ids[:i])
            assert "�" not in d.text and d.text.startswith(seen)
            seen = d.text
        d.finish(ids)
        assert d.text == tok.decode(ids) == text
        cut = ids[: len(ids) - 1]                              # may end inside a character
        d2 = IncrementalDetokenizer(Wrap())
        for j in range(1, len(cut) + 1):
            d2.step(cut[:j])
        d2.finish(cut)
        assert d2.text == tok.decode(cut)


def test_best_of_returns_the_most_likely_samples(llm):
    """``best_of=6, n=2``: six seeded samples run, the two with the best cumulative log-probability come back (they are
    among the six that ``n=6`` gives for the same seed, in order of likelihood); log-probabilities are only returned
    when asked for."""
    from vllm_metax_b200 import SamplingParams

    kw = dict(max_tokens=10, temperature=1.0, seed=5, ignore_eos=True)
    all6 = llm.generate(["Q: ok?"], SamplingParams(n=6, logprobs=0, **kw))[0].outputs
    score = lambda c: sum(e["logprob"] for e in c.logprobs)
    want = sorted(all6, key=lambda c: -score(c))[:2]
    best = llm.generate(["Q: ok?"], SamplingParams(n=2, best_of=6, **kw))[0].outputs
    assert [c.token_ids for c in best] == [c.token_ids for c in want]
    assert [c.index for c in best] == [0, 1] and all(c.logprobs is None for c in best)
    with_lp = llm.generate(["Q: ok?"], SamplingParams(n=1, best_of=6, logprobs=2, **kw))[0].outputs
    assert len(with_lp) == 1 and with_lp[0].token_ids == want[0].token_ids and len(with_lp[0].logprobs[0]["top"]) == 2
    plain = llm.generate(["Q: ok?"], SamplingParams(n=2, best_of=2, **kw))[0].outputs       # best_of == n: nothing to rank
    assert [c.token_ids for c in plain] == [c.token_ids for c in all6[:2]]
