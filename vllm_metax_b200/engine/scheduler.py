"""Continuous-batching scheduler with chunked prefill and recompute preemption.

Every call to ``schedule`` produces one batch under two budgets: at most
``max_num_seqs`` requests and ``max_num_batched_tokens`` new tokens.  Running
requests go first (decodes need one token each), then waiting requests are
admitted while blocks and budget last; a prompt that does not fit the token
budget is split into chunks.  When the pool runs dry the most recently admitted
running request is preempted: its blocks are freed and it re-enters the waiting
queue to be recomputed.  Batches are ordered decode-first so the attention
backend can split the flat token buffer into a decode slice and a prefill slice
(same idea as the batch reordering at
vllm_metax/patch/performance/speculative_decode_perf.py:29-112).
"""
from __future__ import annotations

from collections import deque
from dataclasses import dataclass, field

from ..config import SchedulerConfig
from .block_manager import KVCacheManager
from .sampling_params import Request, RequestStatus


@dataclass
class ScheduledRequest:
    request: Request
    num_new_tokens: int            # tokens fed to the model this step
    start_pos: int                 # position of the first fed token
    samples: bool                  # whether logits of the last fed token are sampled
    num_spec: int = 0              # trailing draft tokens among the fed ones (their logits are verified)
    zombie: bool = False           # the request finished after this step was prepared: the row computes nothing kept

    @property
    def is_decode(self) -> bool:
        return self.num_new_tokens == 1 and self.samples and len(self.request.output_token_ids) > 0


@dataclass
class SchedulerOutput:
    scheduled: list[ScheduledRequest] = field(default_factory=list)
    num_decode: int = 0
    preempted: list[Request] = field(default_factory=list)

    @property
    def num_tokens(self) -> int:
        return sum(s.num_new_tokens for s in self.scheduled)

    @property
    def is_empty(self) -> bool:
        return not self.scheduled


class Scheduler:
    def __init__(self, cfg: SchedulerConfig, kv: KVCacheManager):
        self.cfg = cfg
        self.kv = kv
        self.waiting: deque[Request] = deque()
        self.running: list[Request] = []
        self.paused = False
        self.external_kv = None            # callable(req): attach externally published KV blocks before admission
        # pipelined engine: requests of steps that were launched but whose tokens are not back yet.  They are not
        # scheduled again, not pre-empted, and an abort only marks them (their blocks are in use by the device).
        self.in_flight: set[str] = set()
        self.max_seqs_per_step = cfg.max_num_seqs
        self.num_preemptions = 0
        self.num_draft_tokens = 0
        self.num_accepted_tokens = 0

    # ------------------------------------------------------------------ queue ops
    def add_request(self, req: Request) -> None:
        if req.num_prompt_tokens + req.params.max_tokens > self.cfg.max_model_len:
            req.params.max_tokens = max(1, self.cfg.max_model_len - req.num_prompt_tokens)
        if req.num_prompt_tokens >= self.cfg.max_model_len:
            raise ValueError(f"prompt of {req.num_prompt_tokens} tokens exceeds max_model_len {self.cfg.max_model_len}")
        if self.cfg.policy == "priority":
            self._enqueue_by_priority(req)
        else:
            self.waiting.append(req)

    def _enqueue_by_priority(self, req: Request, front_of_equals: bool = False) -> None:
        """Keep ``waiting`` sorted by (priority, arrival); a pre-empted request goes in front of its equals."""
        key = (req.priority, req.arrival_time)
        i = 0
        for i, other in enumerate(self.waiting):          # queues are short next to a step's cost
            ok = (other.priority, other.arrival_time)
            if ok > key or (front_of_equals and other.priority == req.priority):
                self.waiting.insert(i, req)
                return
        self.waiting.append(req)

    def abort(self, request_id: str) -> bool:
        for q in (self.running, self.waiting):
            for r in list(q):
                if r.request_id == request_id:
                    if request_id in self.in_flight:       # freed by update() when its step comes back
                        r.status = RequestStatus.FINISHED_ABORTED
                        return True
                    q.remove(r)
                    self.kv.free(r)
                    r.status = RequestStatus.FINISHED_ABORTED
                    return True
        return False

    def has_unfinished(self) -> bool:
        return bool(self.waiting or self.running)

    def pause(self) -> None:
        self.paused = True

    def resume(self) -> None:
        self.paused = False

    # ------------------------------------------------------------------ scheduling
    def _preempt_one(self, out: SchedulerOutput, keep: Request) -> bool:
        order = reversed(self.running)
        if self.cfg.policy == "priority":     # the least important request goes first, the latest among equals
            order = sorted(self.running, key=lambda r: (-r.priority, -r.arrival_time))
        for victim in order:
            if victim is keep or victim.request_id in self.in_flight:
                continue
            self.running.remove(victim)
            out.scheduled = [s for s in out.scheduled if s.request is not victim]
            self.kv.free(victim)
            victim.num_computed_tokens = 0
            victim.status = RequestStatus.PREEMPTED
            if self.cfg.policy == "priority":
                self._enqueue_by_priority(victim, front_of_equals=True)
            else:
                self.waiting.appendleft(victim)
            out.preempted.append(victim)
            self.num_preemptions += 1
            return True
        return False

    def schedule(self) -> SchedulerOutput:
        out = SchedulerOutput()
        if self.paused:
            return out
        budget = self.cfg.max_num_batched_tokens
        # ---- running requests (decode, or the next chunk of a long prefill)
        cap = self.max_seqs_per_step
        for req in list(self.running):
            # (a request pre-empted earlier in this pass is no longer running)
            if budget <= 0 or len(out.scheduled) >= cap or (out.preempted and req.status == RequestStatus.PREEMPTED):
                continue
            if req.request_id in self.in_flight or req.finishing:
                continue
            remaining = req.num_tokens - req.num_computed_tokens
            k = len(req.spec_token_ids) if remaining == 1 and req.output_token_ids else 0
            if k and (budget < 1 + k or req.num_tokens + k > self.cfg.max_model_len):
                req.spec_token_ids, k = [], 0       # no room to verify drafts this step
            n = min(remaining, budget) + k
            if not self.cfg.enable_chunked_prefill and n < remaining:
                continue
            ok = True
            need = self.kv.blocks_needed(req, n)
            while need > self.kv.pool.num_free:
                if not self._preempt_one(out, keep=req):
                    ok = False
                    break
            if not ok:
                continue
            if need:
                req.block_ids.extend(self.kv.pool.allocate(need))
            out.scheduled.append(ScheduledRequest(req, n, req.num_computed_tokens, n == remaining + k, k))
            budget -= n
        # ---- admit waiting requests
        while (self.waiting and budget > 0 and len(self.running) < self.cfg.max_num_seqs and not out.preempted
               and len(out.scheduled) < cap):
            req = self.waiting[0]
            if req.finishing:          # pre-empted while its last token was in flight: nothing left to compute
                break
            self.kv.try_prefix_hit(req)
            if self.external_kv is not None and not req.output_token_ids:
                self.external_kv(req)              # KV published by another engine (disaggregated prefill)
            remaining = req.num_tokens - req.num_computed_tokens
            n = min(remaining, budget)
            if not self.cfg.enable_chunked_prefill and n < remaining:
                if not out.scheduled and remaining > self.cfg.max_num_batched_tokens:
                    raise ValueError("prompt longer than max_num_batched_tokens and chunked prefill is off")
                break
            if not self.kv.can_allocate(req, n):
                if req.block_ids:  # drop the prefix-cache references taken above
                    self.kv.free(req)
                    req.num_computed_tokens = 0
                    req.num_cached_tokens = 0
                break
            self.waiting.popleft()
            self.kv.allocate(req, n)
            req.status = RequestStatus.RUNNING
            self.running.append(req)
            out.scheduled.append(ScheduledRequest(req, n, req.num_computed_tokens, n == remaining))
            budget -= n
        # ---- decode-first order
        dec = [s for s in out.scheduled if s.is_decode]
        pre = [s for s in out.scheduled if not s.is_decode]
        out.scheduled = dec + pre
        out.num_decode = len(dec)
        return out

    # ------------------------------------------------------------------ two-phase update (overlapped host work)
    # The engine may prepare step k + 1 on the host while the device still runs step k.  ``begin_step`` applies what
    # step k changes without knowing its tokens (computed-token counts, a provisional output token per sampling
    # request so that the next ``schedule`` sees a decode request); ``finish_step`` puts the real tokens in, checks
    # the stop conditions and retires finished requests.  A request that finishes at step k may already sit in the
    # prepared step k + 1: the engine marks that row (``ScheduledRequest.zombie``) and both phases skip it.
    PROVISIONAL = -1

    def begin_step(self, out: SchedulerOutput) -> None:
        for s in out.scheduled:
            req = s.request
            if s.zombie:
                continue
            assert s.num_spec == 0, "draft verification needs the tokens: not used with overlapped host work"
            req.num_computed_tokens += s.num_new_tokens
            self.kv.commit(req)
            if s.samples:
                req.output_token_ids.append(self.PROVISIONAL)
                if len(req.output_token_ids) >= req.params.max_tokens:
                    req.finishing = True

    def finish_step(self, out: SchedulerOutput, sampled: dict, now: float) -> list[Request]:
        finished = []
        for s in out.scheduled:
            req = s.request
            if s.zombie or not s.samples:
                continue
            tok = sampled[req.request_id]
            req.output_token_ids[-1] = int(tok[0]) if isinstance(tok, (list, tuple)) else int(tok)
            req.token_times.append(now)
            if req.first_token_time is None:
                req.first_token_time = now
            req.finishing = False
            if req.status == RequestStatus.FINISHED_ABORTED:
                continue
            req.check_stop()
            if req.status.finished:
                req.finish_time = now
                if req in self.running:
                    self.running.remove(req)
                else:                       # pre-empted during the overlap window
                    try:
                        self.waiting.remove(req)
                    except ValueError:
                        pass
                self.kv.free(req)
                finished.append(req)
        return finished

    def mark_in_flight(self, out: SchedulerOutput) -> None:
        self.in_flight.update(s.request.request_id for s in out.scheduled)

    def update(self, out: SchedulerOutput, sampled: dict[str, int], now: float) -> list[Request]:
        """Advance request state after the model ran; returns requests that finished."""
        finished = []
        for s in out.scheduled:
            req = s.request
            self.in_flight.discard(req.request_id)
            if req.status == RequestStatus.FINISHED_ABORTED:       # aborted while its step was in flight
                if req in self.running:
                    self.running.remove(req)
                    self.kv.free(req)
                continue
            if s.num_spec:
                # lossless verification of deterministic drafts: the target token of every fed position was
                # sampled; drafts are kept while they equal it, the first mismatch (or the token after the last
                # draft) is the step's own token.  KV of rejected positions is recomputed later.
                targets = sampled[req.request_id]
                drafts = req.spec_token_ids[: s.num_spec]
                acc = 0
                while acc < s.num_spec and drafts[acc] == targets[acc]:
                    acc += 1
                self.num_draft_tokens += s.num_spec
                self.num_accepted_tokens += acc
                req.spec_token_ids = []
                req.num_computed_tokens += 1 + acc
                self.kv.commit(req)
                for tok in targets[: acc + 1]:
                    req.append_token(int(tok), now)
                    req.check_stop()
                    if req.status.finished:
                        break
                if req.status.finished:
                    req.num_computed_tokens = min(req.num_computed_tokens, req.num_tokens)
                    req.finish_time = now
                    self.running.remove(req)
                    self.kv.free(req)
                    finished.append(req)
                continue
            req.num_computed_tokens += s.num_new_tokens
            self.kv.commit(req)
            if s.samples:
                tok = sampled[req.request_id]
                req.append_token(int(tok[0]) if isinstance(tok, (list, tuple)) else tok, now)
                req.check_stop()
                if req.status.finished:
                    req.finish_time = now
                    self.running.remove(req)
                    self.kv.free(req)
                    finished.append(req)
        return finished
