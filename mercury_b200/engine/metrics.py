"""Per-step timing rows and counters (mercury/metrics.py:7-20, :36-112)."""

from __future__ import annotations

from collections import deque
from dataclasses import dataclass


@dataclass(slots=True)
class StepRecord:
    t: float
    num_entries: int
    num_decode: int
    num_tokens: int
    sched_s: float
    step_s: float
    waiting: int
    running: int
    free_pages: int
    preempted: int
    prepare_s: float = 0.0            # host: pages, batch buffer, copy to the device
    kernel_ms: dict | None = None     # per class of kernel call, when the runner times them


def request_record(r) -> dict:
    """One finished (or aborted) request as a row of the metrics; the keys are the
    reference's (mercury/request.py:80-96)."""
    life = r.life
    return {
        "rid": r.rid,
        "arrival": life.arrival,
        "admitted_at": life.first_admission,
        "first_token_at": life.first_token,
        "finished_at": life.end,
        "queue_delay": None if life.first_admission is None else life.first_admission - life.arrival,
        "prompt_tokens": len(r.prompt),
        "output_tokens": len(r.out),
        "cached_tokens": life.cached_tokens,
        "recomputed_tokens": life.computed_tokens,
        "preemptions": life.preemptions,
        "finish_reason": life.end_reason,
        "state": r.state.value,
    }


def percentile(values: list[float], q: float) -> float:
    if not values:
        return 0.0
    ordered = sorted(values)
    pos = (len(ordered) - 1) * q
    low = int(pos)
    high = min(low + 1, len(ordered) - 1)
    return ordered[low] * (1 - (pos - low)) + ordered[high] * (pos - low)


class EngineMetrics:
    def __init__(self, max_steps: int = 500_000):
        self.steps: deque[StepRecord] = deque(maxlen=max_steps)
        self.finished: deque[dict] = deque(maxlen=200_000)
        self.counters = {"steps": 0, "idle_steps": 0, "step_tokens": 0, "decode_tokens": 0,
                         "finished_requests": 0, "aborted_requests": 0, "rejected_requests": 0,
                         "preemptions": 0, "steps_launched_ahead": 0, "surplus_tokens": 0}

    def add_step(self, record: StepRecord) -> None:
        self.steps.append(record)
        self.counters["steps"] += 1
        self.counters["step_tokens"] += record.num_tokens
        self.counters["decode_tokens"] += record.num_decode
        self.counters["preemptions"] += record.preempted

    def summary(self) -> dict:
        step_s = [s.step_s for s in self.steps]
        sched_s = [s.sched_s for s in self.steps]
        total = sum(step_s) or 1e-9
        kernels: dict[str, float] = {}
        for s in self.steps:
            for kind, ms in (s.kernel_ms or {}).items():
                kernels[kind] = kernels.get(kind, 0.0) + ms
        return {**self.counters, "wall_seconds": sum(step_s),
                "prepare_share": sum(s.prepare_s for s in self.steps) / total,
                **({"kernel_ms": {k: round(v, 3) for k, v in sorted(kernels.items())}} if kernels else {}),
                "mean_step_ms": 1e3 * total / max(1, len(step_s)),
                "p50_step_ms": 1e3 * percentile(step_s, 0.5),
                "p99_step_ms": 1e3 * percentile(step_s, 0.99),
                "sched_share": sum(sched_s) / total}
