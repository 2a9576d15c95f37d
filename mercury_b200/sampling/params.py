"""Per-request sampling parameters, with the reference's names and meanings
(mercury/request.py:14-23): greedy iff temperature <= 0; `top_p` nucleus threshold;
`ignore_eos` keeps generating past an end-of-sequence token. `seed` is declared and never
read by the reference; here it keys the request's own random stream."""

from __future__ import annotations

from dataclasses import dataclass


@dataclass
class SamplingParams:
    temperature: float = 0.0
    top_p: float = 1.0
    ignore_eos: bool = False
    seed: int | None = None

    @property
    def greedy(self) -> bool:
        return self.temperature <= 0.0
