"""Per-request timeline on a monotonic clock and the figures derived from it: queue wait, time to
first token, time between tokens, end to end (reference: src/mini_llm_runtime/request_metrics.py:
12-223).  Times are those at which a token became visible to the host, not kernel times."""

from __future__ import annotations

import statistics
from dataclasses import dataclass, field


@dataclass
class RequestTimeline:
    request_id: str
    arrival_ns: int
    prefill_started_ns: list[int] = field(default_factory=list)
    token_ready_ns: list[int] = field(default_factory=list)
    token_ids: list[int] = field(default_factory=list)
    completed_ns: int | None = None

    @property
    def queue_wait_ms(self):
        return None if not self.prefill_started_ns else (self.prefill_started_ns[0] - self.arrival_ns) / 1e6

    @property
    def ttft_ms(self):
        return None if not self.token_ready_ns else (self.token_ready_ns[0] - self.arrival_ns) / 1e6

    @property
    def inter_token_ms(self) -> list[float]:
        return [(b - a) / 1e6 for a, b in zip(self.token_ready_ns, self.token_ready_ns[1:])]

    @property
    def median_tpot_ms(self):
        gaps = self.inter_token_ms
        return statistics.median(gaps) if gaps else None

    @property
    def e2e_ms(self):
        return None if not self.token_ready_ns else (self.token_ready_ns[-1] - self.arrival_ns) / 1e6


class RequestMetricsCollector:
    def __init__(self) -> None:
        self._timelines: dict[str, RequestTimeline] = {}

    def register_request(self, request_id: str, arrival_ns: int) -> None:
        if request_id in self._timelines:
            raise ValueError(f"request {request_id!r} is already registered")
        self._timelines[request_id] = RequestTimeline(request_id, arrival_ns)

    def require_registered(self, request_ids) -> None:
        unknown = [rid for rid in request_ids if rid not in self._timelines]
        if unknown:
            raise KeyError(f"requests without a timeline: {unknown}")

    def record_prefill_started(self, request_id: str, now_ns: int) -> None:
        self._timelines[request_id].prefill_started_ns.append(now_ns)

    def record_tokens(self, emitted, ready_ns: int) -> None:
        for request_id, token in emitted:
            timeline = self._timelines[request_id]
            timeline.token_ready_ns.append(ready_ns)
            timeline.token_ids.append(int(token))

    def record_completed(self, request_ids, now_ns: int) -> None:
        for request_id in request_ids:
            self._timelines[request_id].completed_ns = now_ns

    def get(self, request_id: str) -> RequestTimeline:
        return self._timelines[request_id]

    def summary(self) -> dict:
        def median(values):
            values = [v for v in values if v is not None]
            return statistics.median(values) if values else None

        timelines = list(self._timelines.values())
        return {
            "requests": len(timelines),
            "tokens": sum(len(t.token_ids) for t in timelines),
            "queue_wait_ms_median": median(t.queue_wait_ms for t in timelines),
            "ttft_ms_median": median(t.ttft_ms for t in timelines),
            "tpot_ms_median": median(t.median_tpot_ms for t in timelines),
            "e2e_ms_median": median(t.e2e_ms for t in timelines),
        }
