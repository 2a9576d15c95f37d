"""One request as the scheduler and the engine see it.

Three things live here: what the client asked for (`prompt`, `max_tokens`, sampling), what
has been produced (`out`, with `unread` marking a token that is still on the device), and a
`Lifetime` that books when the request was admitted, preempted and finished. The states are
the reference's (mercury/request.py:7-11): WAITING -> RUNNING -> FINISHED or ABORTED, and
RUNNING -> WAITING when it is preempted. The per-request row of the metrics is put
together in `engine/metrics.py`, not here.
"""

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
class Lifetime:
    """Times (engine clock) and counts of one request's passage through the engine."""

    arrival: float
    first_admission: float | None = None
    last_admission: float | None = None
    first_token: float | None = None
    end: float | None = None
    end_reason: str | None = None
    preemptions: int = 0
    cached_tokens: int = 0        # tokens found in the cache at the last admission
    computed_tokens: int = 0      # tokens this request had to run, recomputation included

    def admit(self, now: float, cached: int, total: int) -> None:
        if self.first_admission is None:
            self.first_admission = now
        self.last_admission = now
        self.cached_tokens = cached
        self.computed_tokens += total - cached

    def preempt(self) -> None:
        self.preemptions += 1
        self.cached_tokens = 0


class Request:
    def __init__(self, rid: str, prompt: list[int], max_tokens: int, arrival: float,
                 hashes: list[int], params: SamplingParams | None = None, seed: int = 0):
        self.rid = rid
        self.prompt = prompt
        self.max_tokens = max_tokens
        self.hashes = hashes                  # chain hashes of the full pages known so far
        self.params = params or SamplingParams()
        self.seed = seed
        self.out: list[int] = []
        # 1 while the last entry of `out` stands for a token that has been sampled on the
        # device and not yet read back (the engine launched the next step ahead of reading it)
        self.unread = 0
        self.seq: Sequence | None = None      # pages and slot while it runs
        self.state = RequestState.WAITING
        self.life = Lifetime(arrival)

    # ---------------------------------------------------------------- tokens

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
        return self.seq_len - self.unread

    @property
    def num_computed(self) -> int:
        return self.seq.num_computed if self.seq is not None else 0

    # ---------------------------------------------------------------- state

    @property
    def arrival(self) -> float:
        return self.life.arrival

    @property
    def num_cached(self) -> int:
        return self.life.cached_tokens

    @property
    def preemptions(self) -> int:
        return self.life.preemptions

    @property
    def finish_reason(self) -> str | None:
        return self.life.end_reason

    @property
    def done(self) -> bool:
        return self.state in (RequestState.FINISHED, RequestState.ABORTED)

    def start_running(self, seq: Sequence, now: float) -> None:
        """Admitted: `seq` holds its pages, of which `seq.num_computed` tokens were cached."""
        self.seq = seq
        self.state = RequestState.RUNNING
        self.life.admit(now, seq.num_computed, self.seq_len)

    def back_to_waiting(self) -> None:
        """Preempted: its pages are gone and it waits again, as a longer prompt."""
        self.seq = None
        self.state = RequestState.WAITING
        self.life.preempt()

    def end(self, state: RequestState, reason: str, now: float | None = None) -> None:
        self.state = state
        self.life.end_reason = reason
        if now is not None:
            self.life.end = now
