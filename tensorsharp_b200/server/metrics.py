"""Process-wide serving counters and their text exposition (``GET /metrics``).

The reference exposes ``/api/queue/status`` and per-request numbers in every final chunk, and no scrape
endpoint (TensorSharp.Server/Endpoints).  A deployment wants the totals too: requests, prompt / generated /
re-used tokens, time spent in prefill and decode, how full the shared steps of the concurrent server run.
Counters are plain numbers under one lock; the exposition is the Prometheus text format, written by hand.
"""
from __future__ import annotations

import threading
from typing import Dict, List, Optional


class ServingMetrics:
    def __init__(self):
        self._lock = threading.Lock()
        self.reset()

    def reset(self) -> None:
        with getattr(self, "_lock", threading.Lock()):
            self.requests = 0
            self.cancelled = 0
            self.prompt_tokens = 0
            self.generated_tokens = 0
            self.kv_reused_tokens = 0
            self.prefill_seconds = 0.0
            self.decode_seconds = 0.0
            self.exchange_recoveries = 0
            self.http: Dict[str, int] = {}

    def record_generation(self, prompt_tokens: int, generated: int, reused: int, prompt_ns: int, eval_ns: int,
                          cancelled: bool = False) -> None:
        with self._lock:
            self.requests += 1
            self.cancelled += 1 if cancelled else 0
            self.prompt_tokens += int(prompt_tokens)
            self.generated_tokens += int(generated)
            self.kv_reused_tokens += int(reused)
            self.prefill_seconds += prompt_ns / 1e9
            self.decode_seconds += eval_ns / 1e9

    def record_exchange_recovery(self) -> None:
        with self._lock:
            self.exchange_recoveries += 1

    def record_http(self, client: Optional[str], status: int) -> None:
        key = f"{client or 'other'}:{status // 100}xx"
        with self._lock:
            self.http[key] = self.http.get(key, 0) + 1

    def render(self, queue=None, gather=None) -> str:
        with self._lock:
            rows: List[str] = []

            def metric(name: str, kind: str, help_: str, value, labels: str = "") -> None:
                if not any(r.startswith(f"# TYPE {name} ") for r in rows):
                    rows.append(f"# HELP {name} {help_}")
                    rows.append(f"# TYPE {name} {kind}")
                rows.append(f"{name}{labels} {value}")
            metric("tensorsharp_generations_total", "counter", "Finished generations (chat and generate).", self.requests)
            metric("tensorsharp_generations_cancelled_total", "counter", "Generations ended by the client going away.", self.cancelled)
            metric("tensorsharp_prompt_tokens_total", "counter", "Prompt tokens of finished generations.", self.prompt_tokens)
            metric("tensorsharp_generated_tokens_total", "counter", "Tokens generated.", self.generated_tokens)
            metric("tensorsharp_kv_reused_tokens_total", "counter", "Prompt tokens served from a session's KV cache.", self.kv_reused_tokens)
            metric("tensorsharp_prefill_seconds_total", "counter", "Time spent preparing prompts.", f"{self.prefill_seconds:.6f}")
            metric("tensorsharp_decode_seconds_total", "counter", "Time spent in token loops.", f"{self.decode_seconds:.6f}")
            metric("tensorsharp_exchange_recoveries_total", "counter",
                   "Requests ended by a device-side wait that gave up, after which the exchanges were rebuilt.", self.exchange_recoveries)
            for key in sorted(self.http):
                client, cls = key.split(":")
                metric("tensorsharp_http_responses_total", "counter", "HTTP responses by client kind and status class.",
                       self.http[key], f'{{client="{client}",status="{cls}"}}')
        if queue is not None:
            st = queue.get_status()
            rows += ["# HELP tensorsharp_queue_pending Requests waiting for a running slot.", "# TYPE tensorsharp_queue_pending gauge",
                     f"tensorsharp_queue_pending {st.pending_requests}",
                     "# HELP tensorsharp_queue_busy 1 while at least one request is running.", "# TYPE tensorsharp_queue_busy gauge",
                     f"tensorsharp_queue_busy {1 if st.busy else 0}",
                     "# HELP tensorsharp_queue_processed_total Requests that held a running slot.",
                     "# TYPE tensorsharp_queue_processed_total counter", f"tensorsharp_queue_processed_total {st.total_processed}"]
        if gather is not None:
            rows += ["# HELP tensorsharp_shared_steps_total Model steps run for concurrent requests.",
                     "# TYPE tensorsharp_shared_steps_total counter", f"tensorsharp_shared_steps_total {gather.steps}",
                     "# HELP tensorsharp_shared_step_rows_total Sequences advanced over all shared steps.",
                     "# TYPE tensorsharp_shared_step_rows_total counter", f"tensorsharp_shared_step_rows_total {gather.step_rows}"]
        return "\n".join(rows) + "\n"


METRICS = ServingMetrics()
