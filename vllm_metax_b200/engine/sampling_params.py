"""Per-request sampling parameters and request/output records."""
from __future__ import annotations

import enum
import time
from dataclasses import dataclass, field
from typing import Optional


@dataclass
class SamplingParams:
    max_tokens: int = 16
    temperature: float = 0.0
    top_k: int = 0
    top_p: float = 1.0
    min_p: float = 0.0
    repetition_penalty: float = 1.0
    presence_penalty: float = 0.0
    frequency_penalty: float = 0.0
    seed: Optional[int] = None
    ignore_eos: bool = False
    stop_token_ids: list[int] = field(default_factory=list)
    min_tokens: int = 0
    logprobs: Optional[int] = None
    n: int = 1                                  # completions per prompt (independent samples; seed + i when seeded)
    best_of: Optional[int] = None               # sample this many (>= n), return the n with the best cumulative log-probability
    stop: list = field(default_factory=list)    # stop STRINGS: generation ends when the output text contains one
    include_stop_str_in_output: bool = False
    bad_words: list = field(default_factory=list)   # strings (need a tokenizer) or token-id lists never to be produced
    skip_special_tokens: bool = True
    truncate_prompt_tokens: Optional[int] = None    # keep only the last k prompt tokens
    # constrained decoding (engine/structured.py)
    allowed_token_ids: Optional[list[int]] = None
    logit_bias: Optional[dict] = None
    guided_choice: Optional[list] = None        # alternatives: token-id lists, or strings with a tokenizer attached
    guided_regex: Optional[str] = None
    guided_json: Optional[object] = None
    guided_grammar: Optional[str] = None        # GBNF / EBNF text with a ``root`` rule (engine/grammar.py)

    def prepare(self, tokenizer=None) -> "SamplingParams":
        """Resolve the constraint once per request (builds the token trie of ``guided_choice``)."""
        if ((self.guided_regex is not None or self.guided_json is not None or self.guided_grammar is not None)
                and getattr(self, "_guide", None) is None):
            from .structured import RegexGuide, schema_to_regex

            if sum(x is not None for x in (self.guided_regex, self.guided_json, self.guided_grammar)) > 1:
                raise ValueError("give one of guided_regex, guided_json, guided_grammar")
            if self.guided_grammar is not None:
                from .grammar import grammar_to_regex

                pattern = grammar_to_regex(self.guided_grammar)
            else:
                pattern = self.guided_regex if self.guided_regex is not None else schema_to_regex(self.guided_json)
            self._guide = RegexGuide(pattern, tokenizer)
        if self.guided_choice is not None and getattr(self, "_trie", None) is None:
            from .structured import TokenTrie, resolve_choices

            self._trie = TokenTrie(resolve_choices(self.guided_choice, tokenizer))
        if self.bad_words and getattr(self, "_bad_seqs", None) is None:
            seqs = []
            for w in self.bad_words:
                if isinstance(w, str):
                    if tokenizer is None:
                        raise ValueError("bad_words given as strings need a tokenizer")
                    # a word is banned with and without a leading space (both tokenisations occur in running text)
                    for form in (w, " " + w.lstrip()):
                        ids = list(tokenizer.encode(form, add_special_tokens=False))
                        if ids and ids not in seqs:
                            seqs.append(ids)
                else:
                    ids = [int(t) for t in w]
                    if ids and ids not in seqs:
                        seqs.append(ids)
            self._bad_seqs = seqs
        return self

    def banned_next_tokens(self, output_token_ids: list) -> list:
        """Tokens that would complete one of the ``bad_words`` sequences given what has been produced."""
        out = []
        for seq in getattr(self, "_bad_seqs", None) or ():
            k = len(seq) - 1
            if k == 0 or (len(output_token_ids) >= k and output_token_ids[-k:] == seq[:-1]):
                out.append(seq[-1])
        return out

    @property
    def constrained(self) -> bool:
        return (bool(self.allowed_token_ids) or bool(self.logit_bias) or self.guided_choice is not None
                or self.guided_regex is not None or self.guided_json is not None or self.guided_grammar is not None
                or bool(self.bad_words))

    @property
    def greedy(self) -> bool:
        return self.temperature <= 0.0

    @property
    def needs_penalties(self) -> bool:
        return self.repetition_penalty != 1.0 or self.presence_penalty != 0.0 or self.frequency_penalty != 0.0


class RequestStatus(enum.Enum):
    WAITING = 0
    RUNNING = 1
    PREEMPTED = 2
    FINISHED_STOPPED = 3
    FINISHED_LENGTH = 4
    FINISHED_ABORTED = 5

    @property
    def finished(self) -> bool:
        return self.value >= 3


class Request:
    """One generation request and its mutable decoding state."""

    __slots__ = ("request_id", "prompt_token_ids", "params", "output_token_ids", "status", "block_ids",
                 "num_computed_tokens", "arrival_time", "first_token_time", "finish_time", "token_times",
                 "eos_token_id", "num_cached_tokens", "logprobs", "prompt", "_hashes", "spec_token_ids", "lora_request", "mm_embeds", "mm_positions", "mm_hash", "_sample_rng", "finishing", "mrope_positions", "mrope_delta", "stop_checker", "stop_reason",
                 "parent_id", "sample_index", "priority")

    def __init__(self, request_id: str, prompt_token_ids: list[int], params: SamplingParams,
                 eos_token_id: Optional[int] = None, prompt: Optional[str] = None,
                 arrival_time: Optional[float] = None):
        self.request_id = request_id
        self._sample_rng = None
        self.stop_checker = None               # StopStringChecker when params.stop is set and a tokenizer is attached
        self.stop_reason = None                # the stop string / stop token id that ended the request
        self.parent_id = None                  # n > 1: the id the samples are reported under ...
        self.sample_index = 0                  # ... and this sample's index
        self.priority = 0                      # scheduling policy "priority": smaller runs first
        self.finishing = False                 # its last token (by length) is being computed: not scheduled again
        self.mrope_positions = None            # [3, prompt] multimodal rotary position streams (Qwen2-VL family) ...
        self.mrope_delta = 0                   # ... and the offset of generated tokens' stream value from their position
        self.prompt_token_ids = list(prompt_token_ids)
        self.params = params
        self.output_token_ids: list[int] = []
        self.status = RequestStatus.WAITING
        self.block_ids: list[int] = []
        self.num_computed_tokens = 0           # tokens whose KV is in the cache
        self.num_cached_tokens = 0             # prefix-cache hits
        self.arrival_time = time.perf_counter() if arrival_time is None else arrival_time
        self.first_token_time: Optional[float] = None
        self.finish_time: Optional[float] = None
        self.token_times: list[float] = []
        self.eos_token_id = eos_token_id
        self.logprobs: list = []
        self.prompt = prompt
        self._hashes: list[int] = []
        self.lora_request = None               # lora.LoRARequest of the adapter this request runs with
        self.mm_embeds = None                  # [n, hidden] encoder features for the prompt's placeholder tokens ...
        self.mm_positions = None               # ... and the (sorted) prompt positions they replace
        self.mm_hash = None                    # content hash of the request's images (salts the prefix-cache keys)
        self.spec_token_ids: list[int] = []     # draft tokens to verify in the next step (speculative decoding)

    @property
    def num_prompt_tokens(self) -> int:
        return len(self.prompt_token_ids)

    @property
    def num_tokens(self) -> int:
        return len(self.prompt_token_ids) + len(self.output_token_ids)

    @property
    def all_token_ids(self) -> list[int]:
        return self.prompt_token_ids + self.output_token_ids

    def token_at(self, i: int) -> int:
        n = len(self.prompt_token_ids)
        return self.prompt_token_ids[i] if i < n else self.output_token_ids[i - n]

    @property
    def is_prefill(self) -> bool:
        """True while the prompt (plus outputs kept across a preemption) is not fully cached."""
        return self.num_computed_tokens < self.num_tokens - 1 or not self.output_token_ids

    def append_token(self, tok: int, now: float) -> None:
        self.output_token_ids.append(tok)
        self.token_times.append(now)
        if self.first_token_time is None:
            self.first_token_time = now

    def check_stop(self) -> None:
        p = self.params
        n_out = len(self.output_token_ids)
        last = self.output_token_ids[-1] if n_out else None
        trie = getattr(p, "_trie", None)
        if trie is not None and n_out and trie.complete(self.output_token_ids):
            self.status = RequestStatus.FINISHED_STOPPED
            return
        guide = getattr(p, "_guide", None)
        if guide is not None and n_out and self.eos_token_id is None and guide.is_complete(guide.text(self.output_token_ids)):
            self.status = RequestStatus.FINISHED_STOPPED      # no end-of-sequence token to ask for: first full match ends
            return
        if n_out >= p.min_tokens and last is not None:
            if (not p.ignore_eos and self.eos_token_id is not None and last == self.eos_token_id) or \
                    last in p.stop_token_ids:
                self.status = RequestStatus.FINISHED_STOPPED
                if last in p.stop_token_ids:
                    self.stop_reason = last
                return
            if self.stop_checker is not None and last >= 0:
                hit = self.stop_checker.step(self.output_token_ids)
                if hit is not None:
                    self.status = RequestStatus.FINISHED_STOPPED
                    self.stop_reason = hit
                    return
        if n_out >= p.max_tokens:
            self.status = RequestStatus.FINISHED_LENGTH


class IncrementalDetokenizer:
    """Text of a growing token sequence without decoding it again from the start.  ``step(ids)`` decodes only the
    tokens since the last stable boundary, with the tokens of the previous step as context (so that tokenizers which
    treat the first token of a call differently - a leading space, for one - give the same text as one full decode),
    and holds tokens back while they end inside a multi-byte character (they decode to U+FFFD until the rest
    arrives).  ``finish(ids)`` emits whatever is still held back."""

    def __init__(self, tokenizer, skip_special_tokens: bool = True):
        self.tok, self.skip = tokenizer, skip_special_tokens
        self.text = ""
        self.prefix = 0          # tokens before this offset are fully emitted ...
        self.read = 0            # ... and tokens [prefix, read) are the context of the next decode

    def _decode(self, ids) -> str:
        return self.tok.decode(list(ids), skip_special_tokens=self.skip)

    def step(self, output_token_ids: list, final: bool = False) -> str:
        ids = output_token_ids
        if len(ids) <= self.read:
            return ""
        before = self._decode(ids[self.prefix:self.read]) if self.read > self.prefix else ""
        now = self._decode(ids[self.prefix:])
        if not final and (len(now) <= len(before) or now.endswith("\ufffd")):
            return ""                     # nothing printable yet (incomplete character): wait for more tokens
        delta = now[len(before):]
        self.prefix, self.read = self.read, len(ids)
        self.text += delta
        return delta

    def finish(self, output_token_ids: list) -> str:
        return self.step(output_token_ids, final=True)


class StopStringChecker:
    """Stop-string search on the incrementally detokenised output of one request.  ``step`` is called after every new
    token with the whole output and searches the tail of the text.  On a hit, ``text`` is cut before the stop string
    (after it with ``include``)."""

    def __init__(self, tokenizer, stops: list, include: bool = False, skip_special_tokens: bool = True):
        self.detok = IncrementalDetokenizer(tokenizer, skip_special_tokens)
        self.stops, self.include = [s for s in stops if s], include
        self.max_len = max((len(s) for s in self.stops), default=0)
        self.text = ""
        self.hit: Optional[str] = None

    def step(self, output_token_ids: list) -> Optional[str]:
        if self.hit is not None:
            return self.hit
        delta = self.detok.step(output_token_ids)
        if not delta:
            return None
        start = max(0, len(self.text) - self.max_len + 1)
        self.text += delta
        best = None
        for s in self.stops:
            i = self.text.find(s, start)
            if i >= 0 and (best is None or i < best[0]):
                best = (i, s)
        if best is None:
            return None
        i, s = best
        self.text = self.text[: i + len(s)] if self.include else self.text[:i]
        self.hit = s
        return s


@dataclass
class CompletionOutput:
    index: int
    token_ids: list[int]
    text: Optional[str]
    finish_reason: Optional[str]
    logprobs: Optional[list] = None
    stop_reason: object = None            # the stop string or stop token id that ended the completion (None: EOS / length)


@dataclass
class RequestMetrics:
    arrival_time: float
    first_token_time: Optional[float]
    finish_time: Optional[float]
    token_times: list[float]

    @property
    def ttft(self) -> Optional[float]:
        return None if self.first_token_time is None else self.first_token_time - self.arrival_time

    @property
    def tpot(self) -> Optional[float]:
        if self.finish_time is None or self.first_token_time is None or len(self.token_times) < 2:
            return None
        return (self.token_times[-1] - self.first_token_time) / (len(self.token_times) - 1)


@dataclass
class RequestOutput:
    request_id: str
    prompt: Optional[str]
    prompt_token_ids: list[int]
    outputs: list[CompletionOutput]
    finished: bool
    metrics: RequestMetrics
    num_cached_tokens: int = 0
