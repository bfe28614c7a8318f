"""Data-parallel serving: ``dp`` independent engine replicas (each with its own scheduler, KV cache and - on a GPU
box - its own device or tensor-parallel group of devices) behind one front that balances requests across them.

    llm = DataParallelLLM(model, data_parallel_size=4, tensor_parallel_size=1, device="cuda", ...)
    outs = llm.generate(prompts, sampling_params)                    # internal load balancing
    outs = llm.generate(prompts, sampling_params, dp_rank=2)         # external: the caller picks the replica

Every replica is a child process running an ordinary single-GPU ``LLM``; requests and results travel over pipes.
(Tensor-parallel replicas are torchrun groups of their own: start one server per group and balance externally, e.g.
by ``dp_rank`` from the caller's side.)  Balancing
is by outstanding work (prompt tokens + tokens still to generate), which is what the replicas' schedulers are
bound by.  A replica that dies turns the calls routed to it into ``EngineDeadError``; the others keep serving.
Parity: the data-parallel deployments the reference's tests drive (tests/v1/test_internal_lb_dp.py,
test_external_lb_dp.py, test_hybrid_lb_dp.py in its tree) and examples/features/data_parallel.
"""
from __future__ import annotations

import multiprocessing as mp
import os
from typing import Optional, Sequence, Union

from .sampling_params import SamplingParams


def _replica_main(rank: int, conn, model, kwargs: dict, visible: Optional[str]) -> None:
    if visible is not None:
        os.environ["CUDA_VISIBLE_DEVICES"] = visible
    os.environ["B200_DP_RANK"] = str(rank)
    try:
        from .llm import LLM

        llm = LLM(model, **kwargs)
        conn.send(("ready", None))
    except BaseException as e:  # noqa: BLE001
        conn.send(("failed", repr(e)))
        return
    while True:
        try:
            msg = conn.recv()
        except EOFError:
            return
        op, payload = msg
        if op == "stop":
            return
        try:
            if op == "generate":
                prompts, sps, extra = payload
                conn.send(("ok", llm.generate(prompts, sps, **extra)))
            elif op == "call":
                name, args, kw = payload
                conn.send(("ok", getattr(llm, name)(*args, **kw)))
        except BaseException as e:  # noqa: BLE001
            conn.send(("error", repr(e)))


class DataParallelLLM:
    def __init__(self, model, data_parallel_size: int = 2, devices_per_replica: int = 1, **llm_kwargs):
        assert data_parallel_size >= 1
        self.dp = 0
        self._model, self._kwargs, self._per = model, dict(llm_kwargs), devices_per_replica
        self._ctx = mp.get_context("spawn")
        self._conns, self._procs, self._load = [], [], []
        self.scale_events: list = []
        self._grow(data_parallel_size)

    # ------------------------------------------------------------------ replicas
    def _visible(self, r: int) -> Optional[str]:
        if self._kwargs.get("device", None) == "cpu":
            return None
        base = os.environ.get("CUDA_VISIBLE_DEVICES")
        if base:
            ids = base.split(",")
        else:
            ids = [str(i) for i in range((r + 1) * self._per)]
        mine = ids[r * self._per:(r + 1) * self._per]
        if len(mine) < self._per:
            raise RuntimeError(f"no devices left for data-parallel replica {r} (visible: {ids})")
        return ",".join(mine)

    def _spawn(self, r: int):
        parent, child = self._ctx.Pipe()
        p = self._ctx.Process(target=_replica_main, args=(r, child, self._model, dict(self._kwargs), self._visible(r)),
                              daemon=True)
        p.start()
        return parent, p

    def _grow(self, new_size: int) -> None:
        started = [(r,) + self._spawn(r) for r in range(self.dp, new_size)]      # all new replicas load at once
        failed = None
        for r, c, p in started:
            try:
                state, info = c.recv()
            except EOFError:
                state, info = "failed", "replica exited while starting"
            if state != "ready":
                failed = failed or f"data-parallel replica {r} failed to start: {info}"
        if failed is not None:
            for _, c, p in started:
                self._stop_one(c, p)
            if self.dp == 0:
                raise RuntimeError(failed)
            raise RuntimeError(failed + f" (still serving with {self.dp} replicas)")
        for r, c, p in started:
            self._conns.append(c)
            self._procs.append(p)
            self._load.append(0)
        self.dp = new_size

    @staticmethod
    def _stop_one(c, p) -> None:
        try:
            c.send(("stop", None))
        except (BrokenPipeError, OSError):
            pass
        p.join(timeout=10)
        if p.is_alive():
            p.terminate()
            p.join(timeout=5)
        c.close()

    def scale(self, new_data_parallel_size: int) -> int:
        """Elastic scaling between calls: start more replicas (they load the model in parallel while the existing
        ones stay up) or retire the highest-numbered ones (their devices are free when this returns).  Calls are
        synchronous, so no request is in flight on a replica that leaves.  Returns the new size.  The use case of
        the reference's examples/ray_serving/elastic_ep/scale.py (``new_data_parallel_size``) for replicas that do
        not share experts."""
        n = int(new_data_parallel_size)
        if n < 1:
            raise ValueError("at least one replica must remain")
        old = self.dp
        if n > old:
            self._grow(n)
        elif n < old:
            for r in range(old - 1, n - 1, -1):
                self._stop_one(self._conns.pop(), self._procs.pop())
                self._load.pop()
            self.dp = n
        if n != old:
            self.scale_events.append((old, n))
        return self.dp

    def heal(self) -> list:
        """Restart replicas whose process has died (same rank, same devices).  Returns the ranks restarted."""
        dead = [r for r, p in enumerate(self._procs) if not p.is_alive()]
        for r in dead:
            self._conns[r].close()
            c, p = self._spawn(r)
            try:
                state, info = c.recv()
            except EOFError:
                state, info = "failed", "replica exited while starting"
            if state != "ready":
                self._stop_one(c, p)
                raise RuntimeError(f"data-parallel replica {r} failed to restart: {info}")
            self._conns[r], self._procs[r], self._load[r] = c, p, 0
        return dead

    # ------------------------------------------------------------------ balancing
    @staticmethod
    def _cost(prompt, sp: SamplingParams) -> int:
        n = len(prompt) if not isinstance(prompt, dict) else len(prompt.get("prompt_token_ids", prompt.get("prompt", "")))
        return n + sp.max_tokens

    def assign(self, prompts: Sequence, sps: Sequence[SamplingParams], dp_rank: Optional[int] = None) -> list[int]:
        """Replica per prompt: the caller's choice, else greedy least-outstanding-work."""
        if dp_rank is not None:
            if not 0 <= dp_rank < self.dp:
                raise ValueError(f"dp_rank {dp_rank} outside [0, {self.dp})")
            return [dp_rank] * len(prompts)
        load = list(self._load)
        out = []
        order = sorted(range(len(prompts)), key=lambda i: -self._cost(prompts[i], sps[i]))   # big requests first
        where = [0] * len(prompts)
        for i in order:
            r = min(range(self.dp), key=lambda k: load[k])
            load[r] += self._cost(prompts[i], sps[i])
            where[i] = r
        out.extend(where)
        return out

    # ------------------------------------------------------------------ API
    def generate(self, prompts: Union[str, Sequence], sampling_params=None, dp_rank: Optional[int] = None, **extra):
        from .llm import EngineDeadError

        if isinstance(prompts, str) or (prompts and isinstance(prompts[0], int)):
            prompts = [prompts]
        n = len(prompts)
        if sampling_params is None or isinstance(sampling_params, SamplingParams):
            sps = [sampling_params or SamplingParams()] * n
        else:
            sps = list(sampling_params)
        where = self.assign(prompts, sps, dp_rank)
        per: dict[int, list[int]] = {}
        for i, r in enumerate(where):
            per.setdefault(r, []).append(i)
        for r in per:                                           # nothing is sent unless every target is alive
            if not self._procs[r].is_alive():
                raise EngineDeadError(f"data-parallel replica {r} is gone")
        for r, idx in per.items():                              # all replicas work at the same time
            self._load[r] += sum(self._cost(prompts[i], sps[i]) for i in idx)
            self._conns[r].send(("generate", ([prompts[i] for i in idx], [sps[i] for i in idx], extra)))
        results: list = [None] * n
        failure = None
        for r, idx in per.items():
            try:
                state, payload = self._conns[r].recv()
            except EOFError:
                state, payload = "error", "replica exited"
            self._load[r] -= sum(self._cost(prompts[i], sps[i]) for i in idx)
            if state != "ok":
                failure = EngineDeadError(f"data-parallel replica {r}: {payload}")
                continue
            for i, o in zip(idx, payload):
                results[i] = o
        if failure is not None:
            raise failure
        self.last_assignment = where
        return results

    def call_all(self, name: str, *args, **kw) -> list:
        """Run ``LLM.<name>(*args, **kw)`` on every replica (sleep, wake_up, update_weights, get_metrics...)."""
        for c in self._conns:
            c.send(("call", (name, args, kw)))
        out = []
        for r, c in enumerate(self._conns):
            state, payload = c.recv()
            if state != "ok":
                raise RuntimeError(f"replica {r}: {payload}")
            out.append(payload)
        return out

    def shutdown(self) -> None:
        for c, p in zip(self._conns, self._procs):
            try:
                c.send(("stop", None))
            except (BrokenPipeError, OSError):
                pass
        for p in self._procs:
            p.join(timeout=10)
            if p.is_alive():
                p.terminate()
        self._conns, self._procs, self._load, self.dp = [], [], [], 0

    def __del__(self):
        try:
            self.shutdown()
        except Exception:
            pass
