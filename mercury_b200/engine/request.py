"""One request's data and its state machine: WAITING -> RUNNING -> FINISHED / ABORTED, and
RUNNING -> WAITING when it is preempted (mercury/request.py:7-11, :26-96)."""

from __future__ import annotations

import enum
from dataclasses import dataclass, field

from ..cache.manager import Sequence
from ..sampling.params import SamplingParams


class RequestState(enum.Enum):
    WAITING = "waiting"
    RUNNING = "running"
    FINISHED = "finished"
    ABORTED = "aborted"


@dataclass
class Request:
    rid: str
    prompt: list[int]
    max_tokens: int
    arrival: float
    hashes: list[int]
    params: SamplingParams = field(default_factory=SamplingParams)
    seed: int = 0

    out: list[int] = field(default_factory=list)
    seq: Sequence | None = None
    num_cached: int = 0
    state: RequestState = RequestState.WAITING
    admitted_at: float | None = None
    last_admitted_at: float | None = None
    first_token_at: float | None = None
    finished_at: float | None = None
    preemptions: int = 0
    recomputed_tokens: int = 0
    finish_reason: str | None = None
    # 1 while the last entry of `out` stands for a token that has been sampled on the
    # device and not yet read back (the engine launched the next step ahead of reading it)
    unread: int = 0

    @property
    def tokens(self) -> list[int]:
        return self.prompt + self.out

    def token_slice(self, start: int, count: int) -> list[int]:
        """tokens[start : start + count] without building the whole list."""
        n = len(self.prompt)
        if start >= n:
            return self.out[start - n:start - n + count]
        if start + count <= n:
            return self.prompt[start:start + count]
        return self.prompt[start:] + self.out[:start + count - n]

    @property
    def seq_len(self) -> int:
        return len(self.prompt) + len(self.out)

    @property
    def known_len(self) -> int:
        """Tokens whose ids the host knows."""
        return len(self.prompt) + len(self.out) - self.unread

    @property
    def num_computed(self) -> int:
        return self.seq.num_computed if self.seq is not None else 0

    @property
    def done(self) -> bool:
        return self.state in (RequestState.FINISHED, RequestState.ABORTED)

    def record(self) -> dict:
        return {
            "rid": self.rid,
            "arrival": self.arrival,
            "admitted_at": self.admitted_at,
            "first_token_at": self.first_token_at,
            "finished_at": self.finished_at,
            "queue_delay": None if self.admitted_at is None else self.admitted_at - self.arrival,
            "prompt_tokens": len(self.prompt),
            "output_tokens": len(self.out),
            "cached_tokens": self.num_cached,
            "recomputed_tokens": self.recomputed_tokens,
            "preemptions": self.preemptions,
            "finish_reason": self.finish_reason,
            "state": self.state.value,
        }
