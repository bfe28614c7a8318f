"""``LLMEngine`` (step loop) and ``LLM`` (offline ``generate`` API).

``LLM(model=<config | path | dict>, ...)`` mirrors the call a vLLM user makes:
``llm.generate(prompts, sampling_params)`` returns one ``RequestOutput`` per prompt with
token ids, text (when a tokenizer is available), finish reason and per-request timing
(TTFT / TPOT).  Sleep / wake, pause / resume and profiling hooks are exposed the way the
reference's examples use them (examples/features/{sleep,pause_resume,profiling}).
"""
from __future__ import annotations

import itertools
import os
import time
from typing import Any, Iterable, Optional, Sequence, Union

import torch

from ..config import CacheConfig, EngineConfig, ModelConfig, ParallelConfig, SchedulerConfig
from .block_manager import KVCacheManager
from .model_runner import ModelRunner
from .sampling_params import (CompletionOutput, Request, RequestMetrics, RequestOutput, RequestStatus,
                              SamplingParams)
from .scheduler import Scheduler


class EngineDeadError(RuntimeError):
    """Raised to every caller once a step failed; the engine refuses further work."""


class LLMEngine:
    def __init__(self, cfg: EngineConfig, tokenizer=None):
        self.cfg = cfg
        self.tokenizer = tokenizer
        self.runner = ModelRunner(cfg)
        nb = self.runner.determine_num_blocks()
        self.runner.init_kv_cache(nb)
        prefix_ok = getattr(self.runner.model, "supports_prefix_caching", True)
        self.kv = KVCacheManager(nb, self.runner.virt_bs, cfg.cache.enable_prefix_caching and prefix_ok)
        self.kv.on_free = [self.runner.release_request]
        self.scheduler = Scheduler(cfg.scheduler, self.kv)
        self.runner.capture_graphs()
        self._ids = itertools.count()
        self.dead: Optional[BaseException] = None
        self.requests: dict[str, Request] = {}
        self.stats = {"steps": 0, "prefill_tokens": 0, "decode_tokens": 0, "preemptions": 0}
        self.step_hooks: list = []
        # pipeline parallel: as many steps in flight as there are stages (B200_PP_OVERLAP=0: lock-step)
        import collections

        from .. import envs
        from ..parallel import state as ps_

        pp_size = ps_.get_pp_group().world_size
        self.pipeline_depth = pp_size if (pp_size > 1 and envs.B200_PP_OVERLAP) else 1
        self.overlap_scheduling = bool(envs.B200_OVERLAP_SCHEDULING) and pp_size == 1
        self._next = None                  # (scheduler output, prepared inputs) of the step prepared ahead of time
        # data-parallel replicas of a MoE model share their experts (DP attention + EP): they step in lock-step
        self._dp_group = ps_.get_dp_group()
        self.dp_sync = self._dp_group.world_size > 1 and cfg.model.is_moe
        if self.dp_sync and pp_size > 1:
            raise ValueError("data-parallel expert sharing is not combined with pipeline parallelism")
        self._inflight: collections.deque = collections.deque()
        if self.pipeline_depth > 1:
            self.scheduler.max_seqs_per_step = max(1, -(-cfg.scheduler.max_num_seqs // self.pipeline_depth))
        from .spec_decode import SpeculativeConfig, make_proposer

        self.spec_config = SpeculativeConfig.from_dict((cfg.additional_config or {}).get("speculative_config"))
        self.proposer = make_proposer(self.spec_config, self)
        if self.proposer is not None:
            from ..parallel import state as ps

            if (ps.get_pp_group().world_size > 1 or self.runner.dcp > 1 or self.runner.pcp > 1
                    or self.runner.state_slots is not None):
                raise ValueError("speculative decoding is not combined with pipeline parallel, decode context parallel "
                                 "or recurrent-state (hybrid) models")
        from ..parallel.liveness import RankLiveness

        self.liveness = RankLiveness.from_default_group()     # None in a single-process engine
        from ..kv_transfer import KVTransferConfig, make_connector

        self.kv_connector = make_connector(
            KVTransferConfig.from_dict((cfg.additional_config or {}).get("kv_transfer_config")), self.runner)
        if self.kv_connector is not None and self.kv_connector.config.is_consumer:
            self.scheduler.external_kv = self._load_external_kv

    # ------------------------------------------------------------------ KV transfer (disaggregated prefill)
    @staticmethod
    def _kv_salt(req: Request):
        salt = None if req.lora_request is None else ("lora", req.lora_request.lora_int_id)
        return salt if req.mm_hash is None else (salt, "mm", req.mm_hash)

    def _load_external_kv(self, req: Request) -> None:
        """Before admission: pull the blocks another engine published for this prompt.  Whatever cannot be loaded
        (missing or corrupt block, no free blocks) is simply recomputed."""
        c, bs = self.kv_connector, self.cfg.cache.block_size
        toks = req.prompt_token_ids
        limit = ((len(toks) - 1) // bs) * bs                       # at least one prompt token is always computed
        have = req.num_computed_tokens
        n = min(c.lookup(toks[:limit], self._kv_salt(req)), limit)
        need = n // bs - len(req.block_ids)
        if n <= have or need > self.kv.pool.num_free:
            return
        req.block_ids.extend(self.kv.pool.allocate(need))
        got = c.load(toks, req.block_ids, n, self._kv_salt(req), first_block=have // bs)
        if got < n:                                                # recompute from the first bad block on
            keep = max(got, have) // bs
            self.kv.pool.release(req.block_ids[keep:])
            del req.block_ids[keep:]
            self.stats["kv_load_failures"] = self.stats.get("kv_load_failures", 0) + 1
        req.num_computed_tokens = max(have, got)
        req.num_cached_tokens = req.num_computed_tokens
        self.stats["kv_external_tokens"] = self.stats.get("kv_external_tokens", 0) + max(0, got - have)

    def _publish_kv(self, so) -> None:
        """After the forward pass, before finished requests give their blocks back: publish the full blocks of
        every prompt whose prefill completed in this step."""
        c, bs = self.kv_connector, self.cfg.cache.block_size
        for s in so.scheduled:
            r = s.request
            if not r.output_token_ids and s.start_pos + s.num_new_tokens >= len(r.prompt_token_ids):
                n = (len(r.prompt_token_ids) // bs) * bs
                if n:
                    c.save(r.prompt_token_ids, r.block_ids, n, self._kv_salt(r))

    # ------------------------------------------------------------------ requests
    def add_request(self, prompt_token_ids: Sequence[int], params: Optional[SamplingParams] = None,
                    request_id: Optional[str] = None, prompt: Optional[str] = None,
                    arrival_time: Optional[float] = None, lora_request=None, multi_modal_data: Optional[dict] = None,
                    priority: int = 0) -> str:
        if self.dead is not None:
            raise EngineDeadError(str(self.dead))
        rid = request_id or f"req-{next(self._ids)}"
        mm = None
        if multi_modal_data is None and params is not None:
            multi_modal_data = getattr(params, "_multi_modal_data", None)   # set by front ends that only pass params through
        if multi_modal_data:
            prompt_token_ids, mm = self.runner.encode_multimodal(list(prompt_token_ids), multi_modal_data)
        if params is not None and params.constrained:
            params.prepare(self.tokenizer)
        if params is not None and params.truncate_prompt_tokens:
            prompt_token_ids = list(prompt_token_ids)[-int(params.truncate_prompt_tokens):]
        req = Request(rid, list(prompt_token_ids), params or SamplingParams(), self.cfg.model.eos_token_id, prompt,
                      arrival_time)
        if params is not None and params.stop:
            if self.tokenizer is None:
                raise ValueError("stop strings need a tokenizer (use stop_token_ids with token-id prompts)")
            from .sampling_params import StopStringChecker

            req.stop_checker = StopStringChecker(self.tokenizer, list(params.stop), params.include_stop_str_in_output,
                                                 params.skip_special_tokens)
        req.priority = int(priority or getattr(params, "_priority", 0) or 0)
        if mm is not None:
            req.mm_embeds, req.mm_positions, req.mm_hash = mm[:3]
            if len(mm) > 3 and mm[3]:
                req.mrope_positions, req.mrope_delta = mm[3]["mrope_positions"], int(mm[3]["mrope_delta"])
        if lora_request is None and params is not None:
            lora_request = getattr(params, "_lora_request", None)      # set by front ends that only pass params through
        if lora_request is not None:
            if getattr(self.runner, "lora", None) is None:
                raise ValueError("the engine was built without enable_lora=True")
            req.lora_request = lora_request
        self.scheduler.add_request(req)
        self.requests[rid] = req
        return rid

    def abort_request(self, request_id: str) -> bool:
        self.requests.pop(request_id, None)
        return self.scheduler.abort(request_id)

    def has_unfinished_requests(self) -> bool:
        return self.scheduler.has_unfinished()

    # ------------------------------------------------------------------ stepping
    def step(self) -> list[Request]:
        """One scheduler iteration; returns the requests that finished in it."""
        if self.dead is not None:
            raise EngineDeadError(str(self.dead))
        if self.pipeline_depth > 1:
            return self._step_pipelined()
        if self._overlap_ok():
            return self._step_overlapped()
        self._next = None
        so = self.scheduler.schedule()
        if self.dp_sync:
            # replicas whose experts span all of them step together: one without work runs a padding token through
            # the model so that every rank joins the step's token exchanges
            busy = self._dp_group.all_gather_object(not so.is_empty)
            if not any(busy):
                if self.scheduler.has_unfinished() and not self.scheduler.paused:
                    raise RuntimeError("scheduler made no progress: KV cache too small for the waiting request")
                return []
            if so.is_empty:
                if self.scheduler.has_unfinished() and not self.scheduler.paused:
                    raise RuntimeError("scheduler made no progress: KV cache too small for the waiting request")
                self.runner.execute_dummy()
                self.stats["dp_padding_steps"] = self.stats.get("dp_padding_steps", 0) + 1
                self._eplb_step()
                return []
        if so.is_empty:
            if self.scheduler.has_unfinished() and not self.scheduler.paused:
                raise RuntimeError("scheduler made no progress: KV cache too small for the waiting request")
            return []
        try:
            if self.liveness is not None:
                self.liveness.check()          # a peer whose step raised: stop before launching work that waits for it
            for hook in self.step_hooks:
                hook("before", self.stats["steps"])
            sampled = self.runner.execute(so)
            for hook in self.step_hooks:
                hook("after", self.stats["steps"])
        except BaseException as e:  # a failed step poisons the engine (memory is released)
            self.dead = e
            if self.liveness is not None:
                self.liveness.announce_failure(repr(e))
            self._release_all()
            raise EngineDeadError(f"engine step failed: {e!r}") from e
        if self.kv_connector is not None and self.kv_connector.config.is_producer:
            self._publish_kv(so)
        now = time.perf_counter()
        finished = self.scheduler.update(so, sampled, now)
        if self.proposer is not None:
            self._propose_drafts(so, sampled)
        self._eplb_step()
        self.stats["steps"] += 1
        self.stats["decode_tokens"] += so.num_decode
        self.stats["prefill_tokens"] += so.num_tokens - so.num_decode
        self.stats["preemptions"] = self.scheduler.num_preemptions
        for r in finished:
            self.requests.pop(r.request_id, None)
        return finished

    def _overlap_ok(self) -> bool:
        """Host work of the next step may run while the device computes this one: plain steps only (no drafts to
        verify, no adapters to route, no recurrent state slots, no replicas or stages to keep in step, no KV
        hand-over)."""
        r = self.runner
        return (self.overlap_scheduling and not self.scheduler.paused and self.proposer is None and not self.dp_sync
                and self.kv_connector is None and r.state_slots is None and r.lora is None and r.dcp == 1 and r.pcp == 1
                and not self.step_hooks and not getattr(r, "keep_hidden", False) and not r.uses_mrope)

    def _step_overlapped(self) -> list[Request]:
        """One step with the host work of the NEXT step (scheduling, staging buffers) done while the device runs this
        one.  The scheduler advances in two phases around it (``Scheduler.begin_step`` / ``finish_step``); a request
        that turns out to have finished stays in the prepared step as a row that writes and returns nothing."""
        sch, runner = self.scheduler, self.runner
        if self._next is not None:
            so, prep = self._next
            self._next = None
        else:
            so = sch.schedule()
            if so.is_empty:
                if sch.has_unfinished() and not sch.paused:
                    raise RuntimeError("scheduler made no progress: KV cache too small for the waiting request")
                return []
            prep = runner.prepare_step(so)
        try:
            if self.liveness is not None:
                self.liveness.check()
            launched = runner.launch_step(prep)
            sch.begin_step(so)
            so2 = sch.schedule()
            prep2 = None if so2.is_empty else runner.prepare_step(so2)
            sampled = launched.result()
        except BaseException as e:
            self.dead = e
            if self.liveness is not None:
                self.liveness.announce_failure(repr(e))
            self._next = None
            self._release_all()
            raise EngineDeadError(f"engine step failed: {e!r}") from e
        finished = sch.finish_step(so, sampled, time.perf_counter())
        self._eplb_step()
        self._next = None if prep2 is None else (so2, prep2)
        if prep2 is not None and all(s.request.status.finished for s in so2.scheduled):
            self._next = None              # everything in the prepared step has just finished: nothing to run
        self.stats["steps"] += 1
        self.stats["decode_tokens"] += so.num_decode
        self.stats["prefill_tokens"] += so.num_tokens - so.num_decode
        self.stats["preemptions"] = sch.num_preemptions
        self.stats["overlapped_steps"] = self.stats.get("overlapped_steps", 0) + (1 if prep2 is not None else 0)
        for r in finished:
            self.requests.pop(r.request_id, None)
        return finished

    def _step_pipelined(self) -> list[Request]:
        """Pipeline parallel with one step per stage in flight: launch steps over disjoint request sets until the
        pipeline is full, then take the oldest step's tokens.  Every stage runs this loop on the same scheduler
        state, so all of them launch the same steps in the same order."""
        try:
            if self.liveness is not None:
                self.liveness.check()
            while len(self._inflight) < self.pipeline_depth:
                so = self.scheduler.schedule()
                if so.is_empty:
                    break
                self.scheduler.mark_in_flight(so)
                for hook in self.step_hooks:
                    hook("before", self.stats["steps"] + len(self._inflight))
                self._inflight.append((so, self.runner.execute_async(so)))
                self.stats["max_inflight"] = max(self.stats.get("max_inflight", 0), len(self._inflight))
            if not self._inflight:
                if self.scheduler.has_unfinished() and not self.scheduler.paused:
                    raise RuntimeError("scheduler made no progress: KV cache too small for the waiting request")
                return []
            so, pending = self._inflight.popleft()
            sampled = pending.result()
            for hook in self.step_hooks:
                hook("after", self.stats["steps"])
        except BaseException as e:
            self.dead = e
            if self.liveness is not None:
                self.liveness.announce_failure(repr(e))
            self._inflight.clear()
            self.scheduler.in_flight.clear()
            self._release_all()
            raise EngineDeadError(f"engine step failed: {e!r}") from e
        if self.kv_connector is not None and self.kv_connector.config.is_producer:
            self._publish_kv(so)
        finished = self.scheduler.update(so, sampled, time.perf_counter())
        self._eplb_step()
        self.stats["steps"] += 1
        self.stats["decode_tokens"] += so.num_decode
        self.stats["prefill_tokens"] += so.num_tokens - so.num_decode
        self.stats["preemptions"] = self.scheduler.num_preemptions
        for r in finished:
            self.requests.pop(r.request_id, None)
        return finished

    def _eplb_step(self) -> None:
        """Expert load balancing: one tick per executed step on every rank (the ranks of an EP group run the same
        steps), between steps; every ``eplb_step_interval`` ticks the experts are re-placed (parallel/eplb.py)."""
        e = self.runner.eplb
        if e is not None and e.step():
            self.stats["eplb_rearrangements"] = e.rearrangements
            if e.last_balancedness is not None:
                self.stats["eplb_balancedness_before"], self.stats["eplb_balancedness_after"] = e.last_balancedness

    def _propose_drafts(self, so, sampled=None) -> None:
        """Attach draft tokens to the requests that will decode next step."""
        self.stats["draft_tokens"] = self.scheduler.num_draft_tokens
        self.stats["accepted_tokens"] = self.scheduler.num_accepted_tokens
        if hasattr(self.proposer, "after_step"):       # model-based proposers draft the whole batch at once
            self.proposer.after_step(so, sampled or {})
            return
        k = self.spec_config.num_speculative_tokens
        for s in so.scheduled:
            r = s.request
            if r.status.finished or not r.output_token_ids or r.num_computed_tokens != r.num_tokens - 1:
                continue
            room = min(k, r.params.max_tokens - len(r.output_token_ids) - 1)
            if room <= 0:
                continue
            if hasattr(self.proposer, "propose_for_request"):
                drafts = self.proposer.propose_for_request(r, room)
            else:
                drafts = self.proposer.propose(r.all_token_ids)
            r.spec_token_ids = [int(t) for t in drafts[:room]]
        self.stats["draft_tokens"] = self.scheduler.num_draft_tokens
        self.stats["accepted_tokens"] = self.scheduler.num_accepted_tokens

    def _release_all(self) -> None:
        for r in list(self.scheduler.running) + list(self.scheduler.waiting):
            self.kv.free(r)
        self.scheduler.running.clear()
        self.scheduler.waiting.clear()

    def make_output(self, r: Request) -> RequestOutput:
        text = None
        if r.stop_checker is not None and r.stop_checker.hit is not None:
            text = r.stop_checker.text             # cut at the stop string
        elif self.tokenizer is not None:
            text = self.tokenizer.decode(r.output_token_ids, skip_special_tokens=r.params.skip_special_tokens)
        reason = {RequestStatus.FINISHED_STOPPED: "stop", RequestStatus.FINISHED_LENGTH: "length",
                  RequestStatus.FINISHED_ABORTED: "abort"}.get(r.status)
        return RequestOutput(r.request_id, r.prompt, r.prompt_token_ids,
                             [CompletionOutput(r.sample_index, list(r.output_token_ids), text, reason,
                                               list(r.logprobs) if r.params.logprobs is not None else None,
                                               r.stop_reason)],
                             r.status.finished,
                             RequestMetrics(r.arrival_time, r.first_token_time, r.finish_time, list(r.token_times)),
                             r.num_cached_tokens)


def _resolve_model(model: Union[str, dict, ModelConfig], **overrides) -> tuple[ModelConfig, Any]:
    tokenizer = None
    if isinstance(model, ModelConfig):
        mc = model
        for k, v in overrides.items():
            setattr(mc, k, v)
        mc.__post_init__()
    elif isinstance(model, dict):
        mc = ModelConfig.from_hf_dict(model, **overrides) if "hidden_size" in model and "architectures" in model \
            else ModelConfig(**{**model, **overrides})
    elif isinstance(model, str) and model.endswith(".gguf"):       # llama.cpp single-file checkpoint
        from .gguf import config_from_gguf, read_gguf

        meta, infos, _ = read_gguf(model)
        mc = ModelConfig.from_hf_dict(config_from_gguf(meta, infos), model_path=model, **overrides)
    else:
        mc = ModelConfig.from_pretrained(model, **overrides)
        try:
            from transformers import AutoTokenizer

            tokenizer = AutoTokenizer.from_pretrained(model)
        except Exception:
            tokenizer = None
    return mc, tokenizer


class LLM:
    """Offline inference entry point.

    >>> llm = LLM(model_config, tensor_parallel_size=1, max_model_len=2048)
    >>> outs = llm.generate([[1, 2, 3]], SamplingParams(max_tokens=8))
    """

    def __init__(self, model: Union[str, dict, ModelConfig], *, tensor_parallel_size: int = 1,
                 pipeline_parallel_size: int = 1, data_parallel_size: int = 1, enable_expert_parallel: bool = False,
                 dtype: Any = None, quantization: Optional[str] = None, kv_cache_dtype: str = "auto",
                 block_size: int = 64, max_model_len: int = 4096, max_num_seqs: int = 256,
                 max_num_batched_tokens: int = 8192, gpu_memory_utilization: float = 0.88,
                 num_gpu_blocks: Optional[int] = None, enable_prefix_caching: bool = False,
                 enable_chunked_prefill: bool = True, enforce_eager: bool = False, device: Optional[str] = None,
                 load_format: str = "auto", seed: int = 0, tokenizer: Any = None, enable_sleep_mode: bool = False,
                 additional_config: Optional[dict] = None, speculative_config: Optional[dict] = None,
                 enable_lora: bool = False, max_loras: int = 4, max_lora_rank: int = 64,
                 kv_transfer_config: Optional[dict] = None, decode_context_parallel_size: int = 1,
                 prefill_context_parallel_size: int = 1, enable_eplb: bool = False, num_redundant_experts: int = 0,
                 eplb_step_interval: int = 3000, eplb_window: int = 1000, use_sequence_parallel_moe: bool = False,
                 all2all_backend: str = "fused_nvlink", scheduling_policy: str = "fcfs"):
        overrides = {"seed": seed}
        if enable_lora:
            overrides.update(enable_lora=True, max_loras=max_loras, max_lora_rank=max_lora_rank)
        if dtype is not None:
            overrides["dtype"] = dtype
        if quantization is not None:
            overrides["quantization"] = quantization
        mc, tok = _resolve_model(model, **overrides)
        if device is None:
            device = "cuda" if torch.cuda.is_available() else "cpu"
        cfg = EngineConfig(
            model=mc,
            cache=CacheConfig(block_size=block_size, num_gpu_blocks=num_gpu_blocks,
                              gpu_memory_utilization=gpu_memory_utilization, kv_cache_dtype=kv_cache_dtype,
                              enable_prefix_caching=enable_prefix_caching),
            parallel=ParallelConfig(tensor_parallel_size, pipeline_parallel_size, data_parallel_size,
                                    enable_expert_parallel, decode_context_parallel_size,
                                    prefill_context_parallel_size, enable_eplb=enable_eplb,
                                    num_redundant_experts=num_redundant_experts,
                                    eplb_step_interval=eplb_step_interval, eplb_window=eplb_window,
                                    use_sequence_parallel_moe=use_sequence_parallel_moe,
                                    all2all_backend=all2all_backend),
            scheduler=SchedulerConfig(max_num_seqs=max_num_seqs, max_num_batched_tokens=max_num_batched_tokens,
                                      max_model_len=max_model_len, enable_chunked_prefill=enable_chunked_prefill,
                                      policy=scheduling_policy),
            device=device, enforce_eager=enforce_eager, load_format=load_format,
            additional_config=dict(additional_config or {},
                                   **({"speculative_config": speculative_config} if speculative_config else {}),
                                   **({"kv_transfer_config": kv_transfer_config} if kv_transfer_config else {})))
        self.config = cfg
        self.engine = LLMEngine(cfg, tokenizer or tok)
        self.tokenizer = self.engine.tokenizer
        self.foreign_finished: list = []       # see _run_capturing
        # B200_PRECISION_DUMP_DIR: record statistics of every module output of this engine's forwards into
        # <dir>/dump_rank<r>.jsonl (utils/precision_dump.py; compare two runs with compare_dumps)
        from .. import envs

        self._precision_dump = None
        if envs.B200_PRECISION_DUMP_DIR:
            from ..parallel import state as ps
            from ..utils.precision_dump import PrecisionDump

            os.makedirs(envs.B200_PRECISION_DUMP_DIR, exist_ok=True)
            path = os.path.join(envs.B200_PRECISION_DUMP_DIR, f"dump_rank{ps.global_rank()}.jsonl")
            self._precision_dump = PrecisionDump(self.engine.runner.model, path)
            self._precision_dump.__enter__()
            import atexit

            atexit.register(self._precision_dump.__exit__)     # flush and close the file when the process ends
            self.engine.runner.use_graphs = False          # module hooks do not run inside a replayed graph

    # ------------------------------------------------------------------ generate
    def _to_ids(self, p) -> tuple[list[int], Optional[str]]:
        if isinstance(p, str):
            if self.tokenizer is None:
                raise ValueError("text prompt given but no tokenizer is available")
            return self.tokenizer.encode(p), p
        if isinstance(p, dict):
            if "prompt_token_ids" in p:
                return list(p["prompt_token_ids"]), p.get("prompt")
            return self._to_ids(p["prompt"])
        return list(p), None

    def generate(self, prompts: Union[str, Sequence], sampling_params: Union[SamplingParams, Sequence[SamplingParams], None] = None,
                 use_tqdm: bool = False, lora_request=None) -> list[RequestOutput]:
        """``lora_request``: one ``LoRARequest`` for all prompts, or a list with one entry (or None) per prompt."""
        if isinstance(prompts, str) or (prompts and isinstance(prompts[0], int)):
            prompts = [prompts]
        n = len(prompts)
        if sampling_params is None or isinstance(sampling_params, SamplingParams):
            sps = [sampling_params or SamplingParams()] * n
        else:
            sps = list(sampling_params)
        now = time.perf_counter()
        import copy

        groups: list[list[str]] = []          # per prompt: the request ids of its sp.n samples
        first_params: dict = {}               # first request id of a group -> the caller's SamplingParams
        reqs: dict[str, Request] = {}
        loras = lora_request if isinstance(lora_request, (list, tuple)) else [lora_request] * n
        for p, sp, lr in zip(prompts, sps, loras):
            ids, text = self._to_ids(p)
            mm = p.get("multi_modal_data") if isinstance(p, dict) else None       # {"image": tensor | PIL | list}
            keep = max(1, int(getattr(sp, "n", 1) or 1))
            k = max(keep, int(getattr(sp, "best_of", None) or 0))
            rids = []
            for i in range(k):
                spi = copy.copy(sp)
                if k > 1:       # independent samples of one prompt (they share its cached prefix when that is on)
                    spi.n, spi.best_of = 1, None
                    spi.seed = None if sp.seed is None else sp.seed + i
                if k > keep and spi.logprobs is None:
                    spi.logprobs = 0            # the chosen tokens' log-probabilities rank the samples
                rid = self.engine.add_request(ids, spi, prompt=text, arrival_time=now, lora_request=lr,
                                              multi_modal_data=mm)
                reqs[rid] = self.engine.requests[rid]
                reqs[rid].sample_index = i
                rids.append(rid)
            groups.append(rids)
            first_params[rids[0]] = sp
        total = len(reqs)

        def merged(rids: list[str]) -> RequestOutput:
            outs = [self.engine.make_output(reqs[r]) for r in rids]
            first = outs[0]
            for o in outs[1:]:
                first.outputs.extend(o.outputs)
                first.finished = first.finished and o.finished
            sp0 = first_params[rids[0]]
            keep = max(1, int(getattr(sp0, "n", 1) or 1))
            if len(first.outputs) > keep:        # best_of: the ``n`` samples with the best cumulative log-probability
                ranked = sorted(first.outputs, key=lambda c: -sum(e["logprob"] for e in (c.logprobs or [])))[:keep]
                for i, c in enumerate(ranked):
                    c.index = i
                    if sp0.logprobs is None:
                        c.logprobs = None
                first.outputs = ranked
            return first

        done: dict[str, Request] = {}
        if self.engine.dp_sync:
            # keep stepping (padding steps once this replica is done) until every replica has finished its prompts
            while any(self.engine._dp_group.all_gather_object(len(done) < total and self.engine.has_unfinished_requests())):
                for r in self.engine.step():
                    if r.request_id in reqs:
                        done[r.request_id] = r
            return [merged(g) for g in groups]
        while len(done) < total:
            for r in self.engine.step():
                if r.request_id in reqs:
                    done[r.request_id] = r
            if not self.engine.has_unfinished_requests() and len(done) < total:
                break
        return [merged(g) for g in groups]

    def beam_search(self, prompts: Union[str, Sequence], beam_width: int = 4, max_tokens: int = 16,
                    length_penalty: float = 1.0, ignore_eos: bool = False) -> list:
        """Beam search per prompt: every round extends all live beams by one token (one batched ``generate`` call
        with ``max_tokens=1`` and the ``2 * beam_width`` most likely continuations; the prompt and the shared beam
        prefixes are served from the prefix cache when it is on), keeps the ``beam_width`` best by cumulative
        log-probability, and moves beams that produced the end-of-sequence token to the finished pool.  Returns, per
        prompt, ``[{"token_ids", "text", "cum_logprob", "score"}, ...]`` best first; ``score`` is the cumulative
        log-probability over ``len ** length_penalty``.  (Upstream's ``LLM.beam_search`` contract.)"""
        if isinstance(prompts, str) or (prompts and isinstance(prompts[0], int)):
            prompts = [prompts]
        eos = self.engine.cfg.model.eos_token_id
        results = []
        sp = SamplingParams(max_tokens=1, temperature=0.0, logprobs=2 * beam_width, ignore_eos=True)

        def score(cum: float, n: int) -> float:
            return cum / (max(n, 1) ** length_penalty)

        for p in prompts:
            base, _ = self._to_ids(p)
            live = [([], 0.0)]                       # (generated tokens, cumulative log-probability)
            finished = []
            for _ in range(max_tokens):
                if not live:
                    break
                outs = self.generate([list(base) + toks for toks, _ in live], sp)
                cand = []
                for (toks, cum), o in zip(live, outs):
                    for t, lp in o.outputs[0].logprobs[0]["top"]:
                        cand.append((toks + [t], cum + lp))
                cand.sort(key=lambda c: -c[1])
                live = []
                for toks, cum in cand:
                    if not ignore_eos and eos is not None and toks[-1] == eos:
                        finished.append((toks, cum))
                    else:
                        live.append((toks, cum))
                    if len(live) >= beam_width:
                        break
                # a finished beam that already beats every live one cannot be overtaken (log-probabilities only fall)
                if finished and live and len(finished) >= beam_width and \
                        max(score(c, len(t)) for t, c in finished) >= max(score(c, len(t)) for t, c in live) \
                        and length_penalty <= 1.0:
                    break
            pool = finished + live
            pool.sort(key=lambda b: -score(b[1], len(b[0])))
            tok = self.tokenizer
            results.append([{"token_ids": t, "text": tok.decode(t, skip_special_tokens=True) if tok is not None else None,
                             "cum_logprob": c, "score": score(c, len(t))} for t, c in pool[:beam_width]])
        return results

    # ------------------------------------------------------------------ chat / pooling / scoring
    def chat(self, messages, sampling_params: Optional[SamplingParams] = None,
             add_generation_prompt: bool = True) -> list[RequestOutput]:
        """``messages``: one conversation (list of ``{"role", "content"}``) or a list of conversations.  Uses the
        tokenizer's chat template when it has one, else a plain ``role: content`` transcript."""
        if messages and isinstance(messages[0], dict):
            messages = [messages]
        prompts = []
        for conv in messages:
            tok = self.tokenizer
            if tok is not None and getattr(tok, "chat_template", None):
                prompts.append(tok.apply_chat_template(conv, tokenize=False, add_generation_prompt=add_generation_prompt))
            else:
                text = "".join(f"{m['role']}: {m['content']}\n" for m in conv)
                prompts.append(text + ("assistant:" if add_generation_prompt else ""))
        return self.generate(prompts, sampling_params)

    def _run_capturing(self, prompts, visit) -> None:
        """Prefill ``prompts`` (one generated token each) and hand ``visit(index, hidden_rows, is_last_chunk)`` the
        final-layer hidden states of every prompt chunk as it is computed."""
        runner = self.engine.runner
        ids = [self._to_ids(p)[0] for p in prompts]
        rid_to_idx = {}
        for i, t in enumerate(ids):
            rid_to_idx[self.engine.add_request(t, SamplingParams(max_tokens=1, ignore_eos=True))] = i
        prev_keep, orig = getattr(runner, "keep_hidden", False), runner.execute
        runner.keep_hidden = True

        def execute(so):
            out = orig(so)
            h, md, _ = runner.last_step
            qsl = md.query_start_loc[: len(so.scheduled) + 1].tolist()
            for j, s in enumerate(so.scheduled):
                i = rid_to_idx.get(s.request.request_id)
                if i is not None and not isinstance(h, dict):
                    last = s.start_pos + s.num_new_tokens >= len(s.request.prompt_token_ids)
                    visit(i, h[qsl[j]: qsl[j + 1]], last)
            return out

        runner.execute = execute
        use_graphs, runner.use_graphs = runner.use_graphs, False      # every step must expose its hidden states
        try:
            while any(r in self.engine.requests for r in rid_to_idx):
                for r in self.engine.step():
                    if r.request_id not in rid_to_idx:        # a generation request of a serving front end that
                        self.foreign_finished.append(r)       # finished during these steps: handed back to it
        finally:
            runner.execute, runner.keep_hidden, runner.use_graphs = orig, prev_keep, use_graphs

    def embed(self, prompts: Union[str, Sequence], pooling: str = "last", normalize: bool = True) -> torch.Tensor:
        """Sentence embeddings ``[n, hidden]`` (fp32, on CPU): the final hidden state of the last prompt token
        (``pooling="last"``) or the mean over all prompt tokens (``"mean"``)."""
        if isinstance(prompts, str) or (prompts and isinstance(prompts[0], int)):
            prompts = [prompts]
        assert pooling in ("last", "mean")
        n = len(prompts)
        acc: list = [None] * n
        cnt = [0] * n

        def visit(i, rows, is_last):
            rows = rows.float()
            if pooling == "last":
                if is_last:
                    acc[i] = rows[-1].cpu()
            else:
                part = rows.sum(0).cpu()
                acc[i] = part if acc[i] is None else acc[i] + part
                cnt[i] += rows.shape[0]

        self._run_capturing(prompts, visit)
        e = torch.stack([a if pooling == "last" else a / max(1, c) for a, c in zip(acc, cnt)])
        return torch.nn.functional.normalize(e, dim=-1) if normalize else e

    encode = embed

    def prompt_logprobs(self, prompts: Union[str, Sequence], top: int = 0) -> list:
        """Log-probability the model assigns to every prompt token given the tokens before it (the ``prompt_logprobs``
        of upstream's sampling parameters; what perplexity / scoring harnesses read).  Per prompt a list with one
        entry per position: ``None`` for the first token, then ``{"token_id", "logprob", "top": [(id, lp), ...]}``.
        The hidden states of every prefill chunk go through the LM head as they are computed, so nothing of size
        ``[prompt, vocab]`` is kept."""
        if isinstance(prompts, str) or (prompts and isinstance(prompts[0], int)):
            prompts = [prompts]
        ids = [self._to_ids(p)[0] for p in prompts]
        out: list = [[None] for _ in ids]
        pos = [0] * len(ids)
        model = self.engine.runner.model

        def visit(i, rows, is_last):
            n0, toks = pos[i], ids[i]
            n = min(rows.shape[0], len(toks) - 1 - n0)          # row j predicts token n0 + j + 1
            pos[i] = n0 + rows.shape[0]
            if n <= 0:
                return
            lp = torch.log_softmax(model.compute_logits(rows[:n]).float(), dim=-1)
            nxt = torch.as_tensor(toks[n0 + 1: n0 + 1 + n], dtype=torch.int64, device=lp.device)
            chosen = lp.gather(1, nxt[:, None])[:, 0].cpu().tolist()
            tv, ti = (lp.topk(min(top, lp.shape[1]), dim=-1) if top > 0 else (None, None))
            tv = tv.cpu().tolist() if tv is not None else None
            ti = ti.cpu().tolist() if ti is not None else None
            for j in range(n):
                out[i].append({"token_id": toks[n0 + 1 + j], "logprob": float(chosen[j]),
                               "top": [(int(a), float(b)) for a, b in zip(ti[j], tv[j])] if top > 0 else []})

        self._run_capturing(ids, visit)
        return out

    def score(self, text_1: Union[str, Sequence], text_2: Union[str, Sequence], pooling: str = "last") -> list[float]:
        """Cosine similarity of the embeddings of ``text_1`` (one prompt, or one per pair) and every ``text_2``."""
        one = isinstance(text_1, str) or (text_1 and isinstance(text_1[0], int))
        a = self.embed([text_1] if one else text_1, pooling)
        many = not (isinstance(text_2, str) or (text_2 and isinstance(text_2[0], int)))
        b = self.embed(text_2 if many else [text_2], pooling)
        if a.shape[0] == 1:
            a = a.expand(b.shape[0], -1)
        return (a * b).sum(-1).tolist()

    def classify(self, prompts: Union[str, Sequence], class_token_ids: Sequence[int]) -> torch.Tensor:
        """Zero-shot classification: the next-token distribution restricted to one token per class,
        ``[n, len(class_token_ids)]`` probabilities."""
        if isinstance(prompts, str) or (prompts and isinstance(prompts[0], int)):
            prompts = [prompts]
        model = self.engine.runner.model
        ids = torch.tensor(list(class_token_ids), dtype=torch.long)
        out: list = [None] * len(prompts)

        def visit(i, rows, is_last):
            if is_last:
                logits = model.compute_logits(rows[-1:]).float()[0].cpu()
                out[i] = torch.softmax(logits[ids], -1)

        self._run_capturing(prompts, visit)
        return torch.stack(out)

    # ------------------------------------------------------------------ weight sync (RLHF loops)
    def update_weights(self, named_tensors) -> int:
        """Load new values for (a subset of) the model's weights from ``(hf_name, tensor)`` pairs through the model's
        own loader (fused / sharded parameters are handled as at start-up).  Returns the number of tensors consumed.
        Captured CUDA graphs stay valid: parameters are updated in place."""
        model = self.engine.runner.model
        pairs = list(named_tensors.items() if isinstance(named_tensors, dict) else named_tensors)
        with torch.no_grad():
            model.load_weights(iter(pairs))
        if self.engine.kv.enable_prefix_caching:
            self.engine.kv.reset_prefix_cache()
        return len(pairs)

    def collective_rpc(self, method: str, args: tuple = (), kwargs: Optional[dict] = None):
        """Call ``method`` on this rank's model runner (every rank of an SPMD engine makes the same call)."""
        return [getattr(self.engine.runner, method)(*args, **(kwargs or {}))]

    # ------------------------------------------------------------------ control surface
    def pause_generation(self) -> None:
        self.engine.scheduler.pause()

    def resume_generation(self) -> None:
        self.engine.scheduler.resume()

    def sleep(self, level: int = 1) -> None:
        from ..device_allocator.cumem import get_mem_allocator_instance

        get_mem_allocator_instance().sleep(("weights",) if level == 1 else tuple())

    def wake_up(self, tags: Optional[list[str]] = None) -> None:
        from ..device_allocator.cumem import get_mem_allocator_instance

        get_mem_allocator_instance().wake_up(tags)

    def start_profile(self, trace_dir: str = "./b200_trace") -> None:
        self._prof = torch.profiler.profile(
            activities=[torch.profiler.ProfilerActivity.CPU] +
                       ([torch.profiler.ProfilerActivity.CUDA] if torch.cuda.is_available() else []),
            on_trace_ready=torch.profiler.tensorboard_trace_handler(trace_dir))
        self._prof.start()

    def stop_profile(self) -> None:
        if getattr(self, "_prof", None) is not None:
            self._prof.stop()
            self._prof = None

    def get_metrics(self) -> dict:
        e = self.engine
        return {**e.stats, "kv_cache_usage": e.kv.usage, "num_running": len(e.scheduler.running),
                "num_waiting": len(e.scheduler.waiting)}
