"""Asynchronous front of ``LLMEngine`` for serving: one background thread steps the engine, request
coroutines receive incremental outputs through per-request queues.

The engine thread is the only code that touches the scheduler / model runner; producers hand requests
over through a lock-protected inbox, so no engine state is shared with the event loop.  A failed step
marks the engine dead: every in-flight and every later request receives ``EngineDeadError``.
Parity: the role of vLLM's AsyncLLM / EngineCore client that the reference serves through
(``vllm serve`` with the platform plugin).
"""
from __future__ import annotations

import asyncio
import threading
import time
from dataclasses import dataclass, field
from typing import AsyncIterator, Optional, Sequence

from ..engine.llm import LLM, EngineDeadError
from ..engine.sampling_params import SamplingParams


@dataclass
class StreamChunk:
    request_id: str
    new_token_ids: list[int]
    token_ids: list[int]
    text: Optional[str]
    finished: bool
    finish_reason: Optional[str] = None
    prompt_tokens: int = 0
    error: Optional[BaseException] = None
    ttft: Optional[float] = None
    logprobs: Optional[list] = None          # entries of the tokens so far (requests with ``logprobs``)


@dataclass
class _Stream:
    queue: asyncio.Queue
    loop: asyncio.AbstractEventLoop
    sent: int = 0
    t_arrival: float = field(default_factory=time.perf_counter)
    t_first: Optional[float] = None
    t_last: Optional[float] = None                 # time of the previous token batch (inter-token latency)
    wall_arrival: float = field(default_factory=time.time)
    traceparent: Optional[str] = None
    params: Optional[SamplingParams] = None
    detok: Optional[object] = None                 # IncrementalDetokenizer of this stream's text


class AsyncLLM:
    def __init__(self, llm: LLM, tracer=None):
        """``tracer``: a ``utils.observability.RequestTracer`` (one span per finished request) or None."""
        from ..utils.observability import latency_histograms

        self.llm = llm
        self.engine = llm.engine
        self.tracer = tracer
        self.histograms = latency_histograms()
        self._inbox: list[tuple] = []
        self._aborts: list[str] = []
        self._calls: list[tuple] = []          # (callable, future, loop): work that must run on the engine thread
        self._lock = threading.Lock()
        self._wake = threading.Event()
        self._streams: dict[str, _Stream] = {}
        self._stop = False
        self._seq = 0
        self.metrics = {"requests_total": 0, "requests_finished": 0, "requests_aborted": 0, "generated_tokens": 0,
                        "prompt_tokens": 0, "ttft_sum": 0.0, "ttft_count": 0}
        self._thread = threading.Thread(target=self._run, name="b200-engine", daemon=True)
        self._thread.start()

    # ------------------------------------------------------------------ engine thread
    def _post(self, st: _Stream, chunk: StreamChunk) -> None:
        st.loop.call_soon_threadsafe(st.queue.put_nowait, chunk)

    def _fail_all(self, err: BaseException) -> None:
        for rid, st in list(self._streams.items()):
            self._post(st, StreamChunk(rid, [], [], None, True, "error", error=err))
        self._streams.clear()

    def _run(self) -> None:
        eng = self.engine
        while not self._stop:
            with self._lock:
                inbox, self._inbox = self._inbox, []
                aborts, self._aborts = self._aborts, []
            for rid in aborts:
                eng.abort_request(rid)
                st = self._streams.pop(rid, None)
                if st is not None:
                    self.metrics["requests_aborted"] += 1
                    self._post(st, StreamChunk(rid, [], [], None, True, "abort"))
            for rid, ids, params, prompt, st in inbox:
                try:
                    eng.add_request(ids, params, request_id=rid, prompt=prompt)
                    self._streams[rid] = st
                    self.metrics["requests_total"] += 1
                    self.metrics["prompt_tokens"] += len(ids)
                except BaseException as e:
                    self._post(st, StreamChunk(rid, [], [], None, True, "error", error=e))
            with self._lock:
                calls, self._calls = self._calls, []
            for fn, fut, loop in calls:
                # e.g. embeddings: the call steps the engine itself until its own requests are done; generation
                # requests that finish meanwhile come back through ``llm.foreign_finished``
                try:
                    res, exc = fn(), None
                except BaseException as e:  # noqa: BLE001
                    res, exc = None, e
                loop.call_soon_threadsafe(self._resolve, fut, res, exc)
                foreign, self.llm.foreign_finished = self.llm.foreign_finished, []
                self._dispatch(foreign)
            if not eng.has_unfinished_requests() or eng.scheduler.paused:
                self._wake.wait(timeout=0.05)
                self._wake.clear()
                continue
            try:
                finished = eng.step()
            except BaseException as e:
                self._fail_all(e if isinstance(e, EngineDeadError) else EngineDeadError(repr(e)))
                continue
            self._dispatch(finished)

    @staticmethod
    def _resolve(fut, res, exc) -> None:
        if fut.cancelled():
            return
        if exc is not None:
            fut.set_exception(exc)
        else:
            fut.set_result(res)

    def _dispatch(self, finished) -> None:
        """Post the new tokens of every stream (and the final chunk of the requests in ``finished``)."""
        eng = self.engine
        now = time.perf_counter()
        done = {r.request_id: r for r in finished}
        for rid, st in list(self._streams.items()):
            r = done.get(rid) or eng.requests.get(rid)
            if r is None:
                continue
            n = len(r.output_token_ids)
            fin = rid in done
            if n == st.sent and not fin:
                continue
            if st.t_first is None and n > 0:
                st.t_first = now
                self.metrics["ttft_sum"] += now - st.t_arrival
                self.metrics["ttft_count"] += 1
                self.histograms["ttft"].observe(now - st.t_arrival)
            elif n > st.sent and st.t_last is not None:
                for _ in range(n - st.sent):
                    self.histograms["itl"].observe((now - st.t_last) / (n - st.sent))
            if n > st.sent:
                st.t_last = now
            new = list(r.output_token_ids[st.sent:n])
            self.metrics["generated_tokens"] += len(new)
            st.sent = n
            out = eng.make_output(r) if fin else None
            if r.stop_checker is not None:
                if fin:
                    text = out.outputs[0].text
                else:     # hold back what could still turn out to be the beginning of a stop string
                    t, hold = r.stop_checker.text, r.stop_checker.max_len - 1
                    text = t[: max(0, len(t) - hold)] if hold > 0 else t
            elif eng.tokenizer is None:
                text = None
            else:
                # one incremental decode per step and stream (decoding the whole output every step would grow
                # quadratically with its length, on the thread that launches the engine's steps)
                if st.detok is None:
                    from ..engine.sampling_params import IncrementalDetokenizer

                    st.detok = IncrementalDetokenizer(eng.tokenizer, r.params.skip_special_tokens)
                st.detok.step(r.output_token_ids, final=fin)
                text = st.detok.text
            self._post(st, StreamChunk(rid, new, list(r.output_token_ids), text, fin,
                                       out.outputs[0].finish_reason if out else None, len(r.prompt_token_ids),
                                       ttft=None if st.t_first is None else st.t_first - st.t_arrival,
                                       logprobs=list(r.logprobs) if r.params.logprobs is not None else None))
            if fin:
                self.metrics["requests_finished"] += 1
                self.histograms["e2e"].observe(now - st.t_arrival)
                if self.tracer is not None:
                    self.tracer.finish(rid, arrival_wall=st.wall_arrival, t_arrival=st.t_arrival, t_first=st.t_first,
                                       t_end=now, prompt_tokens=len(r.prompt_token_ids), completion_tokens=n,
                                       params=st.params, finish_reason=out.outputs[0].finish_reason,
                                       traceparent=st.traceparent, cached_tokens=r.num_cached_tokens)
                del self._streams[rid]


    async def call(self, fn):
        """Run ``fn()`` on the engine thread between two steps and return its result (pooling requests, anything that
        drives the engine itself)."""
        if self.engine.dead is not None:
            raise EngineDeadError(str(self.engine.dead))
        loop = asyncio.get_running_loop()
        fut = loop.create_future()
        with self._lock:
            self._calls.append((fn, fut, loop))
        self._wake.set()
        return await fut

    # ------------------------------------------------------------------ coroutine API
    async def generate(self, prompt_token_ids: Sequence[int], params: SamplingParams, request_id: Optional[str] = None,
                       prompt: Optional[str] = None, traceparent: Optional[str] = None) -> AsyncIterator[StreamChunk]:
        if self.engine.dead is not None:
            raise EngineDeadError(str(self.engine.dead))
        loop = asyncio.get_running_loop()
        with self._lock:
            self._seq += 1
            rid = request_id or f"cmpl-{self._seq}"
            st = _Stream(asyncio.Queue(), loop, traceparent=traceparent, params=params)
            self._inbox.append((rid, list(prompt_token_ids), params, prompt, st))
        self._wake.set()
        try:
            while True:
                chunk: StreamChunk = await st.queue.get()
                if chunk.error is not None:
                    raise chunk.error
                yield chunk
                if chunk.finished:
                    return
        except (asyncio.CancelledError, GeneratorExit):
            self.abort(rid)
            raise

    def abort(self, request_id: str) -> None:
        with self._lock:
            self._aborts.append(request_id)
        self._wake.set()

    def shutdown(self) -> None:
        self._stop = True
        self._wake.set()
        self._thread.join(timeout=5)

    @property
    def is_dead(self) -> bool:
        return self.engine.dead is not None
