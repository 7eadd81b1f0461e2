"""Batched-decode launch: the part of the reference's continuous-batching
scheduler that drives the decode hot path.

`BatchedDecodeLauncher` keeps what `ContinuousBatchScheduler._decode_batch`
and its run loop do for decode (cacheir/runtime/scheduler.py:160-208, 456-478,
535-543): fork one session per request, prefill it, then advance every active
request one token per round through `run_decode_batch`, take the row argmax,
`% vocab_size`, and retire requests that reached their token budget. Admission
policy (priorities, aging, preemption, back-pressure) is host policy outside the
hot path and is not reproduced; the reference's own scheduler can drive
`B200DecodeRuntime` directly since it only needs the runtime duck type.
"""
from __future__ import annotations

import time
from dataclasses import dataclass, field
from typing import Any


@dataclass
class DecodeMetrics:
    """The decode counters of `SchedulerMetrics` (scheduler.py:36-72)."""

    completed_requests: int = 0
    generated_tokens: int = 0
    prefill_tokens: int = 0
    batched_decode_rounds: int = 0
    batched_decode_tokens: int = 0
    total_decode_batch_ms: float = 0.0
    total_decode_ms: float = 0.0
    total_prefill_ms: float = 0.0


@dataclass
class _Active:
    request_id: str
    runtime: Any
    prompt_ids: list[int]
    max_new_tokens: int
    next_id: int
    generated_ids: list[int] = field(default_factory=list)


def argmax_tokens(logits: Any) -> list[int]:
    """`_argmax_tokens` (scheduler.py:535-543): row argmax of the last position, read back to
    the host. CUDA logits go through the library's argmax kernel; only the ids cross PCIe."""
    last = logits[:, -1]
    if getattr(last, "is_cuda", False):
        from . import ops
        return [int(v) for v in ops.argmax_rows(last.contiguous()).tolist()]
    return [int(v) for v in last.argmax(dim=-1).tolist()]


class BatchedDecodeLauncher:
    def __init__(self, template: Any, *, max_batch_size: int = 4):
        self.template = template
        self.max_batch_size = max(1, int(max_batch_size))
        self.metrics = DecodeMetrics()
        self._pending: list[tuple[str, list[int], int]] = []
        self._counter = 0

    def submit(self, prompt_ids: list[int], *, max_new_tokens: int = 16, request_id: str | None = None) -> str:
        self._counter += 1
        rid = request_id or f"req-{self._counter}"
        self._pending.append((rid, [int(t) for t in prompt_ids], int(max_new_tokens)))
        return rid

    def _prefill(self, rid: str, prompt_ids: list[int], max_new_tokens: int) -> _Active:
        runtime = self.template.fork()
        start = time.perf_counter()
        logits, _ = runtime.prefill_tokens(prompt_ids)
        runtime.synchronize()
        self.metrics.total_prefill_ms += (time.perf_counter() - start) * 1000.0
        self.metrics.prefill_tokens += len(prompt_ids)
        vocab = int(runtime.artifact.config.vocab_size)
        next_id = int(logits[0, -1].argmax().item()) % vocab
        return _Active(rid, runtime, prompt_ids, max_new_tokens, next_id)

    def _decode_batch(self, states: list[_Active]) -> None:
        runtime = states[0].runtime
        sessions = [s.runtime for s in states]
        token_ids = [s.next_id for s in states]
        start = time.perf_counter()
        logits = runtime.run_decode_batch(sessions, token_ids)
        runtime.synchronize()
        elapsed_ms = (time.perf_counter() - start) * 1000.0
        next_ids = argmax_tokens(logits)
        self.metrics.batched_decode_rounds += 1
        self.metrics.batched_decode_tokens += len(states)
        self.metrics.total_decode_batch_ms += elapsed_ms
        self.metrics.total_decode_ms += elapsed_ms * len(states)
        vocab = int(runtime.artifact.config.vocab_size)
        for state, next_id in zip(states, next_ids):
            state.generated_ids.append(state.next_id)
            self.metrics.generated_tokens += 1
            state.next_id = int(next_id) % vocab

    def run_until_complete(self) -> dict[str, list[int]]:
        results: dict[str, list[int]] = {}
        active: list[_Active] = []
        while self._pending or active:
            while self._pending and len(active) < self.max_batch_size:
                active.append(self._prefill(*self._pending.pop(0)))
            ready = [s for s in active if len(s.generated_ids) < s.max_new_tokens]
            if ready:
                self._decode_batch(ready)
            still = []
            for s in active:
                if len(s.generated_ids) >= s.max_new_tokens:
                    results[s.request_id] = s.generated_ids
                    s.runtime.kv_cache.clear()
                    self.metrics.completed_requests += 1
                else:
                    still.append(s)
            active = still
        return results
