"""Request tracing and latency histograms for the serving front.

* ``RequestTracer`` - one span per finished request with the attributes upstream's OpenTelemetry integration
  records (``gen_ai.usage.*``, ``gen_ai.latency.time_to_first_token``, ``gen_ai.latency.e2e`` ...).  Spans are handed
  to an exporter: ``OtlpHttpExporter`` posts OTLP/JSON to ``<endpoint>/v1/traces`` from a background thread (no
  OpenTelemetry SDK needed), or any callable for tests.  Incoming W3C ``traceparent`` headers are continued.
* ``Histogram`` - cumulative buckets rendered in Prometheus text format, with the bucket bounds upstream uses for
  time-to-first-token, inter-token latency and end-to-end latency.
Parity: the observability examples of the reference (examples/observability/opentelemetry/README.md:28-45,
prometheus_grafana dashboards) and its fake-collector test (tests/v1/tracing/test_tracing.py:24-60).
"""
from __future__ import annotations

import json
import os
import queue
import threading
import time
import urllib.request
from typing import Callable, Optional

TTFT_BUCKETS = (0.001, 0.005, 0.01, 0.02, 0.04, 0.06, 0.08, 0.1, 0.25, 0.5, 0.75, 1.0, 2.5, 5.0, 7.5, 10.0, 20.0, 40.0, 80.0)
ITL_BUCKETS = (0.01, 0.025, 0.05, 0.075, 0.1, 0.15, 0.2, 0.3, 0.4, 0.5, 0.75, 1.0, 2.5, 5.0, 7.5, 10.0, 20.0, 40.0, 80.0)
E2E_BUCKETS = (0.3, 0.5, 0.8, 1.0, 1.5, 2.0, 2.5, 5.0, 10.0, 15.0, 20.0, 30.0, 40.0, 50.0, 60.0, 120.0, 240.0, 480.0, 960.0)


class Histogram:
    def __init__(self, name: str, help_: str, buckets):
        self.name, self.help = name, help_
        self.bounds = tuple(buckets)
        self.counts = [0] * (len(self.bounds) + 1)
        self.sum = 0.0
        self.n = 0

    def observe(self, v: float) -> None:
        self.sum += v
        self.n += 1
        for i, b in enumerate(self.bounds):
            if v <= b:
                self.counts[i] += 1
                return
        self.counts[-1] += 1

    def render(self, prefix: str = "b200:") -> str:
        lines = [f"# HELP {prefix}{self.name} {self.help}", f"# TYPE {prefix}{self.name} histogram"]
        acc = 0
        for b, c in zip(self.bounds, self.counts):
            acc += c
            lines.append(f'{prefix}{self.name}_bucket{{le="{b}"}} {acc}')
        lines.append(f'{prefix}{self.name}_bucket{{le="+Inf"}} {self.n}')
        lines.append(f"{prefix}{self.name}_sum {self.sum}")
        lines.append(f"{prefix}{self.name}_count {self.n}")
        return "\n".join(lines)


def latency_histograms() -> dict:
    return {
        "ttft": Histogram("time_to_first_token_seconds", "time to first token", TTFT_BUCKETS),
        "itl": Histogram("inter_token_latency_seconds", "time between output tokens", ITL_BUCKETS),
        "e2e": Histogram("e2e_request_latency_seconds", "request latency, arrival to last token", E2E_BUCKETS),
    }


# ---------------------------------------------------------------------------------------------- tracing
def _hex(n_bytes: int) -> str:
    return os.urandom(n_bytes).hex()


def parse_traceparent(header: Optional[str]) -> tuple[Optional[str], Optional[str]]:
    """W3C trace context ``00-<trace id>-<parent span id>-<flags>`` -> (trace id, parent span id)."""
    if not header:
        return None, None
    parts = header.strip().split("-")
    if len(parts) == 4 and len(parts[1]) == 32 and len(parts[2]) == 16:
        return parts[1], parts[2]
    return None, None


class OtlpHttpExporter:
    """Posts spans as OTLP/JSON; a bounded queue and a daemon thread keep the engine loop free of network waits."""

    def __init__(self, endpoint: str, service_name: str = "vllm_metax_b200", timeout: float = 2.0):
        self.url = endpoint.rstrip("/") + ("" if endpoint.rstrip("/").endswith("/v1/traces") else "/v1/traces")
        self.service_name, self.timeout = service_name, timeout
        self.q: "queue.Queue" = queue.Queue(maxsize=4096)
        self.dropped = 0
        self._t = threading.Thread(target=self._loop, daemon=True)
        self._t.start()

    def __call__(self, span: dict) -> None:
        try:
            self.q.put_nowait(span)
        except queue.Full:
            self.dropped += 1

    def _payload(self, spans: list) -> bytes:
        def attr(k, v):
            if isinstance(v, bool):
                return {"key": k, "value": {"boolValue": v}}
            if isinstance(v, int):
                return {"key": k, "value": {"intValue": str(v)}}
            if isinstance(v, float):
                return {"key": k, "value": {"doubleValue": v}}
            return {"key": k, "value": {"stringValue": str(v)}}

        body = {"resourceSpans": [{
            "resource": {"attributes": [attr("service.name", self.service_name)]},
            "scopeSpans": [{"scope": {"name": "vllm_metax_b200.llm_request"}, "spans": [{
                "traceId": s["trace_id"], "spanId": s["span_id"], "parentSpanId": s.get("parent_span_id") or "",
                "name": s["name"], "kind": 2, "startTimeUnixNano": str(s["start_ns"]), "endTimeUnixNano": str(s["end_ns"]),
                "attributes": [attr(k, v) for k, v in s["attributes"].items()]} for s in spans]}]}]}
        return json.dumps(body).encode()

    def _loop(self) -> None:
        while True:
            batch = [self.q.get()]
            try:
                while len(batch) < 64:
                    batch.append(self.q.get_nowait())
            except queue.Empty:
                pass
            try:
                req = urllib.request.Request(self.url, data=self._payload(batch), headers={"Content-Type": "application/json"})
                urllib.request.urlopen(req, timeout=self.timeout).read()
            except Exception:
                self.dropped += len(batch)

    def flush(self, timeout: float = 5.0) -> None:
        t0 = time.time()
        while not self.q.empty() and time.time() - t0 < timeout:
            time.sleep(0.01)
        time.sleep(0.05)


class RequestTracer:
    def __init__(self, exporter: Callable[[dict], None], model_name: str = ""):
        self.exporter, self.model_name = exporter, model_name
        self.spans = 0

    @classmethod
    def from_endpoint(cls, endpoint: Optional[str], model_name: str = "") -> Optional["RequestTracer"]:
        return cls(OtlpHttpExporter(endpoint), model_name) if endpoint else None

    def finish(self, request_id: str, *, arrival_wall: float, t_arrival: float, t_first: Optional[float], t_end: float,
               prompt_tokens: int, completion_tokens: int, params=None, finish_reason: Optional[str] = None,
               traceparent: Optional[str] = None, cached_tokens: int = 0) -> dict:
        trace_id, parent = parse_traceparent(traceparent)
        attrs = {
            "gen_ai.request.id": request_id, "gen_ai.response.model": self.model_name,
            "gen_ai.usage.prompt_tokens": int(prompt_tokens), "gen_ai.usage.completion_tokens": int(completion_tokens),
            "gen_ai.usage.cached_tokens": int(cached_tokens), "gen_ai.latency.e2e": float(t_end - t_arrival),
        }
        if t_first is not None:
            attrs["gen_ai.latency.time_to_first_token"] = float(t_first - t_arrival)
            if completion_tokens > 1:
                attrs["gen_ai.latency.time_per_output_token"] = float((t_end - t_first) / (completion_tokens - 1))
        if finish_reason:
            attrs["gen_ai.response.finish_reason"] = finish_reason
        if params is not None:
            attrs.update({"gen_ai.request.max_tokens": int(params.max_tokens),
                          "gen_ai.request.temperature": float(params.temperature),
                          "gen_ai.request.top_p": float(params.top_p)})
        start_ns = int(arrival_wall * 1e9)
        span = {"name": "llm_request", "trace_id": trace_id or _hex(16), "span_id": _hex(8), "parent_span_id": parent,
                "start_ns": start_ns, "end_ns": start_ns + int((t_end - t_arrival) * 1e9), "attributes": attrs}
        self.exporter(span)
        self.spans += 1
        return span
